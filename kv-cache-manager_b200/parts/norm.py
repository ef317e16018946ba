"""RMSNorm with the residual add that precedes it fused in.

out = w * round(x * rsqrt(mean(x^2) + eps)); statistics in float32 over the float32 residual
stream (the reference's kernel, ``src/cuda/kernels.cu:34-49``; its separate residual kernel,
``:84-88``, is folded into this one).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import library as K
from .base import NORMS, ClosingNorm, Norm, settle


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, hidden: int, eps: float, init=("ones",)) -> None:
        super().__init__()
        self.hidden, self.eps = hidden, float(eps)
        self.declare("weight", (hidden,), init, "vector")

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        K.rmsnorm(x, pending, self.param("weight"), out, self.eps, rows)


@NORMS.register("rmsnorm_output")
class OutputRMSNorm(Norm):
    """The norm of a block that normalises what a sublayer RETURNS, not what it reads:
    x += mult * w * y / sqrt(mean(y^2) + eps), statistics and sum in float32.  ``forward(x, y, out)``
    adds into the float32 residual ``x`` and, when ``out`` is given, writes the new rows of x in the
    storage dtype for the next sublayer to read."""

    def __init__(self, hidden: int, eps: float, mult: float = 1.0, init=("ones",)) -> None:
        super().__init__()
        self.hidden, self.eps, self.mult = hidden, float(eps), float(mult)
        self.declare("weight", (hidden,), init, "vector")

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], out: Optional[torch.Tensor],
                rows: Optional[torch.Tensor] = None) -> None:
        if rows is not None or pending is None:
            raise ValueError("rmsnorm_output: needs the sublayer's output for every row")
        K.rms_scale_add(x, pending, self.param("weight"), out, self.eps, self.mult)


@NORMS.register("dyt")
class DynamicTanh(Norm):
    """A norm without statistics: out = b + w * tanh(alpha x); alpha is one learned number, w and b
    are vectors.  ``pending`` is what the layer before left to be added to the stream first: None,
    one float32 tensor, or a list of (float32 tensor, scale) pairs (a block whose sublayers' outputs
    are summed hands them on unsummed); the sum, the stream and the tanh are float32."""

    def __init__(self, hidden: int, init=("ones",)) -> None:
        super().__init__()
        self.hidden = hidden
        self.declare("weight", (hidden,), init, "vector")
        self.declare("bias", (hidden,), ("normal", 0.02), "vector")
        self.declare("alpha", (), ("ones_jitter", 0.1), "vector")
        self._f32 = {}

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        self._f32 = {n: self.param(n).to(device=device, dtype=torch.float32).reshape(-1).contiguous()
                     for n in ("weight", "bias", "alpha")}

    def forward(self, x: torch.Tensor, pending, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        if pending is None:
            pending = []
        elif isinstance(pending, torch.Tensor):
            pending = [(pending if pending.dtype == torch.float32 else pending.float(), 1.0)]
        f = self._f32
        K.dyt_norm(x, pending, f["weight"], f["bias"], f["alpha"], out, rows)


@NORMS.register("rmsnorm_offset")
class OffsetRMSNorm(Norm):
    """RMS norm whose weight is stored as its distance from one: x / sqrt(mean(x^2) + eps) * (1 + w).  The
    multiplier 1 + w is formed once, in float32 (in 16 bits the sum would lose the weight's low bits), and the
    statistics are float32.  As a block's norm it is used in pairs by the "sandwich" block (one closes a sublayer,
    one opens the next: ``kernels.library.norm_post_pre``); ``forward`` is the plain pre-norm, with the row gather
    of a final norm."""

    def __init__(self, hidden: int, eps: float, init=("normal", 0.1)) -> None:
        super().__init__()
        self.hidden, self.eps = hidden, float(eps)
        self.declare("weight", (hidden,), init, "vector")
        self.multiplier: Optional[torch.Tensor] = None

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        self.multiplier = (1.0 + self.param("weight").to(device=device, dtype=torch.float32)).contiguous()

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        if isinstance(pending, ClosingNorm) and pending.eps == self.eps:
            K.norm_post_pre(x, pending.y, pending.multiplier, self.multiplier, out, self.eps, rows)
            return
        settle(x, pending)
        K.norm_post_pre(x, None, None, self.multiplier, out, self.eps, rows)
