"""Arrangement of parts in one layer.  ``PreNormBlock``: x += mixer(norm1(x)); x += ffn(norm2(x))
(``src/model/llama.cpp:104-124``).  The residual stream x is float32; a sub-layer's output is
not added at once but handed on as *pending* and added inside the next norm kernel.
``OutputNormBlock``: x += m * norm1(mixer(x)); x += m * norm2(ffn(x)): the sublayers read the
stream itself and the norms sit on their outputs; nothing is left pending."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import library as K
from .base import BLOCKS, Block, ClosingNorm, FeedForward, Mixer, Norm, SiteCache, StepContext, settle


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward) -> None:
        super().__init__()
        self.norm1 = self.add_child("norm1", norm1)
        self.mixer = self.add_child("mixer", mixer)
        self.norm2 = self.add_child("norm2", norm2)
        self.ffn = self.add_child("ffn", ffn)

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                site: SiteCache) -> torch.Tensor:
        h = torch.empty(x.shape, dtype=ctx.dtype, device=x.device)
        self.norm1.forward(x, pending, h)
        y = self.mixer.forward(h, ctx, site)
        self.norm2.forward(x, y, h)
        return self.ffn.forward(h, ctx)


@BLOCKS.register("output_norm")
class OutputNormBlock(Block):
    """``norm1`` / ``norm2`` are norms of the "rmsnorm_output" kind (they own the residual add and the
    multiplier).  ``ffn`` may be None: a layer of a mixer only.  The sublayers read the stream in the
    storage dtype: with float32 storage that is x itself, else a copy ``ctx.h_stream`` that the norm
    kernels keep current (the embedding may have left one; otherwise the first block makes it)."""

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm] = None,
                 ffn: Optional[FeedForward] = None) -> None:
        super().__init__()
        self.norm1 = self.add_child("norm1", norm1)
        self.mixer = self.add_child("mixer", mixer)
        self.norm2 = self.add_child("norm2", norm2) if norm2 is not None else None
        self.ffn = self.add_child("ffn", ffn) if ffn is not None else None
        if (self.norm2 is None) != (self.ffn is None):
            raise ValueError("output_norm block: a feed-forward and its norm come together")

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                site: SiteCache) -> Optional[torch.Tensor]:
        if pending is not None:
            K.add_residual(x, pending)
        if ctx.dtype == torch.float32:
            h = keep = None
        else:
            h = ctx.h_stream
            if h is None:
                h = ctx.h_stream = torch.empty(x.shape, dtype=ctx.dtype, device=x.device)
                K.cast_rows(x, h)
            keep = h
        self.norm1.forward(x, self.mixer.forward(x if h is None else h, ctx, site), keep)
        if self.ffn is not None:
            self.norm2.forward(x, self.ffn.forward(x if h is None else h, ctx), keep)
        return None


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    """x += mixer(h) + ffn(h) with ONE norm, h = norm1(x): both sublayers read the same normalised rows.
    Their float32 outputs are not summed here: they are handed on as a list of (tensor, scale) pairs and
    added into the stream inside the next norm kernel (a mixer made of several branches returns such a
    list itself).  ``norm1`` must take such a list (the "dyt" norm does).  ``ffn`` may be None."""

    def __init__(self, norm1: Norm, mixer: Mixer, ffn: Optional[FeedForward] = None) -> None:
        super().__init__()
        self.norm1 = self.add_child("norm1", norm1)
        self.mixer = self.add_child("mixer", mixer)
        self.ffn = self.add_child("ffn", ffn) if ffn is not None else None

    def forward(self, x: torch.Tensor, pending, ctx: StepContext, site: SiteCache):
        h = torch.empty(x.shape, dtype=ctx.dtype, device=x.device)
        self.norm1.forward(x, pending, h)
        y = self.mixer.forward(h, ctx, site)
        out = list(y) if isinstance(y, (list, tuple)) else [(y, 1.0)]
        if self.ffn is not None:
            out.append((self.ffn.forward(h, ctx, out_dtype=torch.float32), 1.0))
        return out


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    """Every sublayer normalised on both sides: x += norm1b(mixer(norm1(x))); x += norm2b(ffn(norm2(x))).  The four
    norms expose ``multiplier`` (float32 [hidden]) and ``eps`` ("rmsnorm_offset").  The sublayers return float32; the
    norm that closes one sublayer and the norm that opens the next are one kernel, also across layers: the
    closing norm of a layer's last sublayer is handed on as a ``ClosingNorm`` and applied by whatever reads the
    stream next (the next sandwich block's opening norm, the final norm, or a part between layers through
    ``settle``).  ``fuse`` off: every norm is a launch of its own and the stream is complete when the layer ends.
    ``ffn`` may be None: a layer of a mixer only."""

    def __init__(self, norm1: Norm, mixer: Mixer, norm1b: Norm, norm2: Optional[Norm] = None,
                 ffn: Optional[FeedForward] = None, norm2b: Optional[Norm] = None) -> None:
        super().__init__()
        self.norm1 = self.add_child("norm1", norm1)
        self.mixer = self.add_child("mixer", mixer)
        self.norm1b = self.add_child("norm1b", norm1b)
        self.norm2 = self.add_child("norm2", norm2) if norm2 is not None else None
        self.ffn = self.add_child("ffn", ffn) if ffn is not None else None
        self.norm2b = self.add_child("norm2b", norm2b) if norm2b is not None else None
        if not ((self.norm2 is None) == (self.ffn is None) == (self.norm2b is None)):
            raise ValueError("sandwich block: a feed-forward and its two norms come together")

    def forward(self, x: torch.Tensor, pending, ctx: StepContext, site: SiteCache):
        fuse = ctx.options.get("fuse", True)
        h = torch.empty(x.shape, dtype=ctx.dtype, device=x.device)
        if isinstance(pending, ClosingNorm) and pending.eps == self.norm1.eps:
            K.norm_post_pre(x, pending.y, pending.multiplier, self.norm1.multiplier, h, self.norm1.eps)
        else:
            settle(x, pending)
            K.norm_post_pre(x, None, None, self.norm1.multiplier, h, self.norm1.eps)
        y = self.mixer.forward(h, ctx, site)
        if self.ffn is None:
            return self._close(x, y, self.norm1b, fuse)
        if fuse and self.norm1b.eps == self.norm2.eps:
            K.norm_post_pre(x, y, self.norm1b.multiplier, self.norm2.multiplier, h, self.norm2.eps)
        else:
            K.norm_post_pre(x, y, self.norm1b.multiplier, None, None, self.norm1b.eps)
            K.norm_post_pre(x, None, None, self.norm2.multiplier, h, self.norm2.eps)
        y = self.ffn.forward(h, ctx, out_dtype=torch.float32)
        return self._close(x, y, self.norm2b, fuse)

    @staticmethod
    def _close(x: torch.Tensor, y: torch.Tensor, norm: Norm, fuse: bool):
        if fuse:
            return ClosingNorm(y, norm.multiplier, norm.eps)
        K.norm_post_pre(x, y, norm.multiplier, None, None, norm.eps)
        return None
