"""Gated feed-forward: down( act(x Wg^T) * (x Wu^T) ), gate and up fused into one matrix
[2I, H] (gate rows first) so that one product feeds the activation kernel
(``src/model/llama.cpp:120-122``; activation ``src/cuda/kernels.cu:72-82``).
"""
from __future__ import annotations

import torch

from ..kernels import library as K
from .base import FEED_FORWARDS, FeedForward, StepContext
from .linear import Linear, STREAM_MAX_BYTES, TCGEN05_GATED_MAX_HIDDEN, TCGEN05_MIN_ROWS, tiles_fill_well


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    def __init__(self, hidden: int, intermediate: int, activation: str = "silu") -> None:
        super().__init__()
        if activation != "silu":
            raise ValueError(f"gated_mlp: activation '{activation}' has no kernel (only 'silu')")
        self.hidden, self.intermediate = hidden, intermediate
        self.gate_up = self.add_child("gate_up", Linear(hidden, 2 * intermediate))
        self.down = self.add_child("down", Linear(intermediate, hidden))

    def forward(self, h: torch.Tensor, ctx: StepContext, out_dtype=None) -> torch.Tensor:
        act = torch.empty((h.shape[0], self.intermediate), dtype=h.dtype, device=h.device)
        w = self.gate_up.param("weight")
        # A handful of rows (decode): the gate/up product and the activation in one kernel (the
        # same roundings as the two separate kernels).
        if (h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and ctx.options.get("gemm", "auto") in ("auto", "native")
                and ctx.options.get("fuse", True) and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0
                and K.gate_up_silu_supported(h.shape[0], self.intermediate, h.shape[1])):
            K.gate_up_silu(h, w, act)
        elif (h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and ctx.options.get("fuse", True)
              and ctx.options.get("gemm", "auto") in ("auto", "native", "tcgen05", "pair") and h.shape[0] >= TCGEN05_MIN_ROWS
              and (ctx.options.get("gemm", "auto") != "auto"
                   or (tiles_fill_well(h.shape[0], 2 * self.intermediate, h.device)
                       and h.shape[1] <= TCGEN05_GATED_MAX_HIDDEN))
              and K.tcgen05_gemm_supported(h, w)):
            # Many rows (prefill): the tcgen05 product applies the activation in its epilogue.  It
            # saves the activation kernel (time ~ rows x I) and loses about a tenth of the product
            # against the library (time ~ rows x I x hidden): a win up to a hidden size of ~3,000
            # (TinyLlama shape: 84 us against 76 + 15; Llama-3-8B shape: the library wins).
            # Beyond that size the two-SM form of the kernel is the faster of this engine's two
            # (Llama-3-8B shape: about 0.4 against 0.58 ms).
            if ctx.options.get("gemm", "auto") == "pair" or h.shape[1] > TCGEN05_GATED_MAX_HIDDEN:
                K.gate_up_silu_tcgen05_pair(h, w, act)
            else:
                K.gate_up_silu_tcgen05(h, w, act)
        else:
            K.silu_mul(self.gate_up.forward(h, ctx), act)
        return self.down.forward(act, ctx, out_dtype)


@FEED_FORWARDS.register("dense_mlp")
class DenseMLP(FeedForward):
    """Ungated feed-forward: down( act(x Wu^T) ); act "relu2" = max(z, 0)^2, or "polynorm":
    a N(z) + b N(z^2) + c N(z^3) + e with the four learned numbers ``act`` = (a, b, c, e), powers taken
    element by element and N(v) = v / sqrt(mean(v^2) + norm_eps) over a row's ``intermediate`` values (the up
    product's float32 result goes in; sums and roots are float32)."""

    def __init__(self, hidden: int, intermediate: int, activation: str = "relu2", norm_eps: float = 1e-6) -> None:
        super().__init__()
        if activation not in ("relu2", "polynorm"):
            raise ValueError(f"dense_mlp: activation '{activation}' has no kernel (only 'relu2', 'polynorm')")
        self.hidden, self.intermediate, self.activation, self.norm_eps = hidden, intermediate, activation, float(norm_eps)
        self.up = self.add_child("up", Linear(hidden, intermediate, hidden ** -0.5))
        self.down = self.add_child("down", Linear(intermediate, hidden, intermediate ** -0.5))
        self._coef = None
        if activation == "polynorm":
            self.declare("act", (4,), ("normal", 0.5), "vector")

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        if self.activation == "polynorm":
            self._coef = self.param("act").to(device=device, dtype=torch.float32).contiguous()

    def forward(self, h: torch.Tensor, ctx: StepContext, out_dtype=None) -> torch.Tensor:
        w = self.up.param("weight")
        M = h.shape[0]
        if self.activation == "polynorm":
            z = self.up.forward(h, ctx, out_dtype=torch.float32)
            act = torch.empty((M, self.intermediate), dtype=h.dtype, device=h.device)
            K.poly_norm_act(z, self._coef, act, self.norm_eps)
            return self.down.forward(act, ctx, out_dtype)
        # A handful of rows (decode): the up product applies the activation in its epilogue (the same
        # roundings as the two separate kernels), where `matmul_nt` would take the streaming kernel anyway.
        if (h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and ctx.options.get("gemm", "auto") in ("auto", "native")
                and ctx.options.get("fuse", True) and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0
                and (M <= 8 or w.numel() * 2 <= STREAM_MAX_BYTES) and K.stream_gemm_supported(M, self.intermediate, h.shape[1])):
            z = torch.empty((M, self.intermediate), dtype=h.dtype, device=h.device)
            K.gemm_stream_relu_sq(h, w, z)
        else:
            z = self.up.forward(h, ctx)
            K.relu_sq(z, z)
        return self.down.forward(z, ctx, out_dtype)
