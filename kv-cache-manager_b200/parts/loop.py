"""The entry of a span of layers that runs several times in a row with the same weights.

Before the first layer of every pass t = 0, 1, ... the stream is mixed with the embedding's output x0:

    x <- W_in [x ; x0] + step[t]

W_in [hidden, 2 hidden] (x's columns first), step [passes, hidden].  x0 is what the embedding left in
``ctx.shared[source]`` (float32).  The product's operands are in the storage dtype, its result, the added row
and the new stream are float32.  Every pass is a call site of its own in the run order, so each has its own
cache pages and state rows; this part only rewrites the stream.
"""
from __future__ import annotations

import torch

from ..kernels import library as K
from .base import StepContext, StreamPart, settle
from .linear import Linear


class LoopEntry(StreamPart):
    def __init__(self, hidden: int, passes: int, source: str = "x0") -> None:
        super().__init__()
        self.hidden, self.passes, self.source = hidden, passes, source
        self.inp = self.add_child("inp", Linear(2 * hidden, hidden, (2 * hidden) ** -0.5))
        self.declare("step", (passes, hidden), ("normal", 0.1), "vector")
        self._step = None

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        self._step = self.param("step").to(device=device, dtype=torch.float32).contiguous()

    def forward(self, x: torch.Tensor, pending, ctx: StepContext, arg=None):
        t = int(arg or 0)
        settle(x, pending)
        both = torch.empty((x.shape[0], 2 * self.hidden), dtype=ctx.dtype, device=x.device)
        K.concat_cast(x, ctx.shared[self.source], both)
        y = self.inp.forward(both, ctx, out_dtype=torch.float32)
        K.add_bias_rows(y, self._step[t])
        return y, None
