"""Several residual streams instead of one (hyper-connections).

The model carries ``streams`` copies x_1 .. x_S of the residual stream, [T, S, D] float32, all equal to the
embedding's output at the start.  Every sublayer q of a layer owns three small tensors: ``in`` [S], ``out`` [S] and
``mix`` [S, S] (indexed [from, to]):

    u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_t <- sum_s mix[s, t] x_s + out[t] y   (all t from the old x)

and the model's output is the sum of the streams.  A plain residual stream is the case S = 1, in = out = mix = 1.

Parts: ``StreamsEmbedding`` (the S copies), ``HyperConnection`` (one sublayer's three tensors), the block
``hyper_connection`` and the final norm ``rmsnorm_streams`` (sum of the streams, then an RMS norm, on the wanted
rows only).  The write that ends one sublayer and the read (with its norm) that opens the next are ONE kernel
(``kernels.library.hc_step``), also across layers: a block hands its last sublayer's output on as a
``HyperPending`` and the next reader of the streams applies it.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import library as K
from .base import BLOCKS, NORMS, Block, FeedForward, Mixer, Norm, Part, SiteCache, StepContext


class HyperConnection(Part):
    """The three tensors of one sublayer: how the streams are read, how its output is written, how they mix."""

    def __init__(self, streams: int) -> None:
        super().__init__()
        self.streams = int(streams)
        self.declare("in", (streams,), ("ones_jitter", 0.3), "vector")
        self.declare("out", (streams,), ("ones_jitter", 0.3), "vector")
        self.declare("mix", (streams, streams), ("eye_jitter", 0.2), "vector")
        self.in_w = self.out_w = self.mix_w = None

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        self.in_w, self.out_w, self.mix_w = (self.param(n).to(device=device, dtype=torch.float32).contiguous()
                                             for n in ("in", "out", "mix"))


class HyperPending:
    """A sublayer's float32 output ``y`` (plus an optional bias row) that is still to be written into the streams
    through ``hc``'s mix and out tensors."""
    __slots__ = ("y", "bias", "hc")

    def __init__(self, y: torch.Tensor, bias: Optional[torch.Tensor], hc: HyperConnection) -> None:
        self.y, self.bias, self.hc = y, bias, hc


def hyper_step(x: torch.Tensor, pending: Optional[HyperPending], read: Optional[HyperConnection],
               norm_w: Optional[torch.Tensor], h: Optional[torch.Tensor], eps: float, rows=None,
               in_w: Optional[torch.Tensor] = None) -> None:
    """Applies what is pending to the streams and/or forms the next sublayer's normalised input."""
    if pending is not None and not isinstance(pending, HyperPending):
        raise TypeError("several residual streams: the layer before must hand on a HyperPending (or nothing)")
    if pending is None and h is None:
        return
    p = pending
    K.hc_step(x, p.y if p else None, p.bias if p else None, p.hc.mix_w if p else None, p.hc.out_w if p else None,
              (in_w if in_w is not None else read.in_w) if h is not None else None, norm_w, h, eps, rows)


class StreamsEmbedding(Part):
    """x [T, S, D] float32: every stream starts as the token's row of the table."""

    def __init__(self, vocab: int, hidden: int, streams: int) -> None:
        super().__init__()
        self.vocab, self.hidden, self.streams = vocab, hidden, int(streams)
        self.declare("weight", (vocab, hidden), ("normal", 0.02), "table")

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = torch.empty((ctx.rows, self.streams, self.hidden), dtype=torch.float32, device=ctx.tokens.device)
        K.embed_streams(ctx.tokens, self.param("weight"), x)
        return x


@NORMS.register("rmsnorm_streams")
class StreamsRMSNorm(Norm):
    """The model's last norm over several streams: x = sum of the streams, out = w * x / sqrt(mean(x^2) + eps),
    formed for the wanted rows only; what the last layer left pending is applied on the way."""

    def __init__(self, hidden: int, eps: float, streams: int, init=("ones",)) -> None:
        super().__init__()
        self.hidden, self.eps, self.streams = hidden, float(eps), int(streams)
        self.declare("weight", (hidden,), init, "vector")
        self._w = self._ones = None

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        self._w = self.param("weight").to(device=device, dtype=torch.float32).contiguous()
        self._ones = torch.ones(self.streams, dtype=torch.float32, device=device)

    def forward(self, x: torch.Tensor, pending, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        hyper_step(x, pending, None, self._w, out, self.eps, rows, in_w=self._ones)


@BLOCKS.register("hyper_connection")
class HyperConnectionBlock(Block):
    """Pre-norm layer over several residual streams: the mixer reads norm1(sum_s in1[s] x_s) and writes through
    (mix1, out1); the feed-forward, where the layer has one, likewise with (in2, mix2, out2).  ``norm1``/``norm2`` are
    plain weighted RMS norms ("rmsnorm": ``weight``, ``eps``); their statistics are taken inside the kernel that
    reads the streams.  A mixer with an ``out_bias`` (float32 row added to its output) gets it added in the same
    kernel that writes its output into the streams.  ``ctx.options['fuse']`` off: the streams are complete when the
    layer ends (one more launch a layer)."""

    def __init__(self, streams: int, norm1: Norm, mixer: Mixer, norm2: Optional[Norm] = None,
                 ffn: Optional[FeedForward] = None) -> None:
        super().__init__()
        if (norm2 is None) != (ffn is None):
            raise ValueError("hyper_connection block: a feed-forward and its norm come together")
        self.streams = int(streams)
        self.norm1 = self.add_child("norm1", norm1)
        self.mixer = self.add_child("mixer", mixer)
        self.hc1 = self.add_child("hc1", HyperConnection(streams))
        self.norm2 = self.add_child("norm2", norm2) if norm2 is not None else None
        self.ffn = self.add_child("ffn", ffn) if ffn is not None else None
        self.hc2 = self.add_child("hc2", HyperConnection(streams)) if ffn is not None else None
        self._w1 = self._w2 = None
        if hasattr(mixer, "defer_bias"):
            mixer.defer_bias = True                 # the bias of its output rides in the kernel that writes the streams

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        self._w1 = self.norm1.param("weight").to(device=device, dtype=torch.float32).contiguous()
        if self.norm2 is not None:
            self._w2 = self.norm2.param("weight").to(device=device, dtype=torch.float32).contiguous()

    def forward(self, x: torch.Tensor, pending, ctx: StepContext, site: SiteCache):
        T, _, D = x.shape
        h = torch.empty((T, D), dtype=ctx.dtype, device=x.device)
        hyper_step(x, pending, self.hc1, self._w1, h, self.norm1.eps)
        y = self.mixer.forward(h, ctx, site)
        out = HyperPending(y, getattr(self.mixer, "out_bias", None), self.hc1)
        if self.ffn is not None:
            hyper_step(x, out, self.hc2, self._w2, h, self.norm2.eps)
            out = HyperPending(self.ffn.forward(h, ctx, out_dtype=torch.float32), None, self.hc2)
        if not ctx.options.get("fuse", True):
            hyper_step(x, out, None, None, None, 0.0)
            return None
        return out
