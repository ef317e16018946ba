"""Gated linear attention: a mixer with a fixed-size state per request and a decay for every key channel.

Per head a float32 matrix S [dk, dv], zero at a request's start, is carried from token to token:

    S <- diag(alpha) S + k v^T;    o = S^T q

with q = W_q h * dk^-1/2, k = W_k h (heads x dk), v = W_v h (heads x dv) and the decay of every key channel
alpha = sigmoid(z)^(1/tau), z = W_a2 (W_a1 h) + b (heads x dk; the projection goes through ``decay_rank``
numbers).  Each head's o is divided by its root mean square over dv and multiplied by a weight [dv] shared
by the heads, the heads side by side are multiplied by SiLU(W_g h) and go through the output projection.

State of a request: one float32 row per call site, S of every head.  The recurrence is the engine's
matrix-state scan in its linear form with channel-wise decays (csrc/cuda/delta_rule.cu); the products
return float32 and everything after them (scale, decays, recurrence, norm) is float32 in both storage dtypes.
The first-stage decay projection is padded with zero rows to a multiple of 8 (and W_a2 with matching zero
columns) once after loading, so that the second product reads aligned rows.
"""
from __future__ import annotations

import torch

from ..kernels import library as K
from .base import MIXERS, Mixer, SiteCache, StateSpec, StepContext
from .linear import Linear, matmul_nt


@MIXERS.register("gla")
class GatedLinearAttention(Mixer):
    def __init__(self, hidden: int, heads: int, dk: int, dv: int, decay_rank: int, tau: float, norm_eps: float) -> None:
        super().__init__()
        if not (tau > 0):
            raise ValueError("gla: tau must be positive")
        self.hidden, self.heads, self.dk, self.dv, self.decay_rank = hidden, heads, dk, dv, decay_rank
        self.tau, self.norm_eps = float(tau), float(norm_eps)
        std = hidden ** -0.5
        self.qkv = self.add_child("qkv", Linear(hidden, heads * (2 * dk + dv), std))       # q | k | v, float32 result
        self.g = self.add_child("g", Linear(hidden, heads * dv, std))
        self.a1 = self.add_child("a1", Linear(hidden, decay_rank, std))
        self.a2 = self.add_child("a2", Linear(decay_rank, heads * dk, decay_rank ** -0.5))
        self.o = self.add_child("o", Linear(heads * dv, hidden, (heads * dv) ** -0.5))
        self.declare("a2_bias", (heads * dk,), ("normal", 1.0), "vector")
        self.declare("norm", (dv,), ("ones_jitter", 0.1), "vector")
        self._f32 = {}
        self._a1 = self._a2 = None

    def state_spec(self) -> StateSpec:
        return StateSpec((self.heads * self.dk * self.dv,), torch.float32)

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        if self.dk > K.delta_scan_max_dk():
            raise ValueError(f"gla: key size {self.dk} exceeds the recurrence kernel's {K.delta_scan_max_dk()}")
        self._f32 = {n: self.param(n).to(device=device, dtype=torch.float32).contiguous() for n in self.param_specs()}
        r = (self.decay_rank + 7) // 8 * 8
        a1, a2 = self.a1.param("weight"), self.a2.param("weight")
        if r != self.decay_rank:
            p1 = torch.zeros((r, self.hidden), dtype=a1.dtype, device=a1.device)
            p1[:self.decay_rank] = a1
            p2 = torch.zeros((self.heads * self.dk, r), dtype=a2.dtype, device=a2.device)
            p2[:, :self.decay_rank] = a2
            a1, a2 = p1, p2
        self._a1, self._a2 = a1, a2

    def forward(self, h: torch.Tensor, ctx: StepContext, site: SiteCache) -> torch.Tensor:
        T, H, dk, dv = h.shape[0], self.heads, self.dk, self.dv
        qkv = self.qkv.forward(h, ctx, out_dtype=torch.float32)
        gate = self.g.forward(h, ctx)
        low = matmul_nt(h, self._a1, h.dtype, ctx.options)
        decay = matmul_nt(low, self._a2, torch.float32, ctx.options)                 # becomes alpha in place
        K.gla_prepare(qkv, 0, H * dk, dk ** -0.5, decay, self._f32["a2_bias"], self.tau)
        o = torch.empty((T, H * dv), dtype=torch.float32, device=h.device)           # (the scan zeroes padding rows)
        K.state_scan(K.SCAN_LINEAR_CHANNEL, qkv, (0, H * dk, 2 * H * dk), None, None, decay, site.state, ctx, o, H, H, dk, dv)
        gated = torch.empty((T, H * dv), dtype=h.dtype, device=h.device)
        K.group_rms_gate(o, gate, self._f32["norm"], gated, dv, self.norm_eps, False, "silu")
        return self.o.forward(gated, ctx, out_dtype=torch.float32)
