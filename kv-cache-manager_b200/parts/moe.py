"""A feed-forward of many small gated experts, of which every row uses ``top``.

    z = W_router h (float32);  s = softmax(z) over all experts
    experts form ``groups`` equal groups of neighbours; a group's score is its largest s; only
    experts of the best ``keep`` groups can be chosen; the ``top`` largest s among them win
    y = sum_chosen (scale * s_e) * expert_e(h)  [+ sigmoid(w_sg . h) * shared(h)]
    expert(h) = W_down (silu(W_gate h) * (W_up h)),  no biases; the weights are not renormalised

Options (constructor parameters): ``scores`` "sigmoid" takes s = sigmoid(z) instead of the softmax; ``correction``
declares a learned number per expert that is added to s for the CHOICE only (choice scores may be negative, the
weights use s itself); ``group_top`` = 2 scores a group by the sum of its two largest choice scores;
``shared_gate`` False runs the shared expert ungated (the router matrix then has no extra row).

The experts' matrices are stacked ([E, 2F, D] gate rows before up rows, [E, D, F]); the optional
shared expert is the engine's gated feed-forward and runs for every row; its per-row gate is one
more row of the router matrix.  Routing, the expert products and the weighted sum are this
engine's kernels (csrc/cuda/moe.cu); nothing is read on the host, so steps can be recorded.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import library as K
from .base import FEED_FORWARDS, FeedForward, StepContext
from .mlp import GatedMLP


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, hidden: int, experts: int, expert_ff: int, top: int, scale: float = 1.0, groups: int = 1,
                 keep: int = 1, shared_ff: int = 0, scores: str = "softmax", correction: bool = False, group_top: int = 1,
                 shared_gate: bool = True) -> None:
        super().__init__()
        if experts < 1 or groups < 1 or experts % groups or not (1 <= keep <= groups):
            raise ValueError(f"routed_experts: {experts} experts do not form {groups} equal groups of which {keep} are kept")
        if not (1 <= top <= (experts // groups) * keep):
            raise ValueError(f"routed_experts: top {top} exceeds the {(experts // groups) * keep} experts a row may choose from")
        self.hidden, self.experts, self.expert_ff, self.top = hidden, experts, expert_ff, top
        self.scale, self.groups, self.keep = float(scale), groups, keep
        if scores not in ("softmax", "sigmoid") or group_top not in (1, 2):
            raise ValueError("routed_experts: scores 'softmax' | 'sigmoid', group_top 1 | 2")
        self.scores, self.group_top = scores, int(group_top)
        self.shared_gate = bool(shared_gate) and bool(shared_ff)
        self.shared: Optional[GatedMLP] = None
        if shared_ff:
            self.shared = self.add_child("shared", GatedMLP(hidden, shared_ff))
        # router rows, then (with a shared expert) the row of its gate
        self.declare("router", (experts + (1 if self.shared_gate else 0), hidden), ("normal", hidden ** -0.5), "matrix")
        if correction:
            self.declare("correction", (experts,), ("normal", 0.1), "vector")
        self._correction = None
        self.declare("gate_up", (experts * 2 * expert_ff, hidden), ("normal", hidden ** -0.5), "matrix")
        self.declare("down", (experts * hidden, expert_ff), ("normal", expert_ff ** -0.5), "matrix")
        self._wgu = self._wd = self._router = None

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        E, F, D = self.experts, self.expert_ff, self.hidden
        self._wgu = self.param("gate_up").to(dtype).view(E, 2 * F, D)
        self._wd = self.param("down").to(dtype).view(E, D, F)
        r = self.param("router")
        self._router = r if r.dtype in (torch.float32, dtype) else r.to(dtype)
        if "correction" in self.param_specs():
            self._correction = self.param("correction").to(device=device, dtype=torch.float32).contiguous()

    def forward(self, h: torch.Tensor, ctx: StepContext, out_dtype=None) -> torch.Tensor:
        """Returns float32 rows (``out_dtype`` is accepted for the feed-forward interface and must allow that)."""
        if out_dtype not in (None, torch.float32):
            raise ValueError("routed_experts: the weighted sum is float32")
        M, D, top = h.shape[0], self.hidden, self.top
        dev = h.device
        idx = torch.empty((M, top), dtype=torch.int32, device=dev)
        wt = torch.empty((M, top), dtype=torch.float32, device=dev)
        gate = torch.empty((M,), dtype=torch.float32, device=dev) if self.shared_gate else None
        K.moe_route(h, self._router, self.experts, self.groups, self.keep, top, self.scale, idx, wt, gate, self.scores,
                    self._correction, self.group_top)
        work = torch.empty((K.moe_work_ints(M, top, self.experts),), dtype=torch.int32, device=dev)
        act = torch.empty((M * top, self.expert_ff), dtype=h.dtype, device=dev)
        y = torch.empty((M * top, D), dtype=torch.float32, device=dev)
        xs = None
        if (h.dtype == torch.bfloat16 and ctx.options.get("gemm", "auto") != "plain"
                and K.moe_tcgen05_supported(self.expert_ff, D) and h.stride(0) % 8 == 0):
            xs = torch.empty((M * top, D), dtype=h.dtype, device=dev)        # tensor-core products
        K.moe_experts(h, self._wgu, self._wd, idx, work, act, y, xs)
        shared_y = self.shared.forward(h, ctx, out_dtype=torch.float32) if self.shared is not None else None
        out = torch.empty((M, D), dtype=torch.float32, device=dev)
        K.moe_combine(y, work, wt, self.experts, shared_y, gate, out)
        return out
