"""Grouped-query attention over the paged cache: the mixer of this architecture.

Per step: fused QKV product; rotary encoding of q and k in place and the write of K (encoded)
and V into the rows' page slots (one kernel); attention of every row over its request's pages
(keys up to the row's own position, optionally only the last ``window`` of them); output
product.  Order and formulas after ``src/model/llama.cpp:108-116``; scale = 1/sqrt(head_dim)
unless given.  All rows of a step are written to the cache before any row reads it, so rows of
one portion see each other through the pages and causality is the bound ``position + 1``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import library as K
from .base import CacheSpec, MIXERS, Mixer, PositionEncoding, SiteCache, StepContext
from .linear import Linear, matmul_nt


@MIXERS.register("attention")
class PagedAttention(Mixer):
    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PositionEncoding, window: int = 0, scale: Optional[float] = None) -> None:
        super().__init__()
        if num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        self.hidden, self.nh, self.nkv, self.hd = hidden, num_heads, num_kv_heads, head_dim
        self.window = int(window or 0)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.position = self.add_child("position", position)
        self.qkv = self.add_child("qkv", Linear(hidden, (num_heads + 2 * num_kv_heads) * head_dim))
        self.o = self.add_child("o", Linear(num_heads * head_dim, hidden))

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(self.nkv, self.hd, self.window)

    def forward(self, h: torch.Tensor, ctx: StepContext, site: SiteCache) -> torch.Tensor:
        g = ctx.groups[site.group]
        pos = self.position
        w = self.qkv.param("weight")
        M = h.shape[0]
        # A handful of rows (decode): one kernel does the product, the rotary encoding and the
        # cache write; it gives the same bits as the three separate kernels below.
        if (site.writes and h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and ctx.options.get("gemm", "auto") in ("auto", "native") and ctx.options.get("fuse", True)
                and pos.inv_freq is not None and pos.rotary_dim == self.hd and not pos.interleaved
                and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0
                and K.qkv_rope_cache_supported(M, h.shape[1], self.nh, self.nkv, self.hd)):
            qkv = torch.empty((M, self.nh * self.hd), dtype=h.dtype, device=h.device)
            K.qkv_rope_cache(h, w, qkv, ctx.positions, pos.inv_freq, g.slot_mapping, site.k, site.v,
                             self.nh, self.nkv, self.hd)
        else:
            qkv = self.qkv.forward(h, ctx)
            K.rope_cache(qkv, ctx.positions, pos.inv_freq, pos.rotary_dim, pos.interleaved,
                         g.slot_mapping, site.k, site.v, self.nh, self.nkv, self.hd, g.block_size,
                         write_cache=site.writes)
        out = torch.empty((h.shape[0], self.nh * self.hd), dtype=h.dtype, device=h.device)
        K.paged_attention(qkv, out, site.k, site.v, g.block_tables, ctx, self.nh, self.nkv, self.hd,
                          self.scale, self.window)
        return self.o.forward(out, ctx)


def padded_head_dim(n: int) -> int:
    """The cache's head size for heads of ``n`` elements: the next size that the tensor-core attention
    kernels take (multiples of 16 up to 128, of 32 up to 256), else the next multiple of 8."""
    if n <= 128:
        return (n + 15) // 16 * 16
    if n <= 256:
        return (n + 31) // 32 * 32
    return (n + 7) // 8 * 8


@MIXERS.register("attention_general")
class GeneralAttention(Mixer):
    """Grouped-query softmax attention over the paged cache with the options that other designs add,
    each a constructor parameter:

    * query/key heads of ``dk`` elements and value heads of ``dv`` (the cache's head size is
      ``padded_head_dim(max(dk, dv))``; the elements beyond a head's own are zero, which changes no
      score and leaves the output's extra columns zero; the output product's matrix is padded with
      zero columns once, at load);
    * ``bias``: q, k and v projections with a bias;
    * ``proj_norm``: q <- w_q * q / sqrt(mean(q^2) + eps) over the WHOLE q projection (all heads at
      once), k likewise, before the rotation;
    * a rotary ``position`` that may cover only the first dimensions of a head, in rotate-half or in
      interleaved pairs;
    * ``rotate_values``: every value is turned by its own position over all ``dv`` dimensions (frequencies
      base^(-2m/dv) with the position encoding's base, the same pairing) before it is cached, and a head's
      output at position i (the weighted sum of the turned values) is turned back by -i;
    * ``head_norm``: q and k of every head scaled to unit root mean square (no weights), after the
      rotation;
    * ``softcap``: score <- cap * tanh(score / cap) after the scale;
    * ``window``: row i sees keys j with 0 <= i - j < window; with ``keep_first`` > 0 also every j < keep_first
      (j <= i), at its true position.  Such a mixer asks for pages that are never given back: the cache
      manager's windows release pages from the front, where the kept keys lie;
    * ``sink``: a learned number per head whose exponential joins the softmax's denominator (no key, no
      value, not scaled, not capped);
    * ``value_mix``: "source" leaves this layer's values (as projected) in ``ctx.shared[mix_key]`` for later
      layers of the same step; "mix" replaces v by v + lambda (v_source - v) before it is cached.

    Projection, norms, rotation, mixing and the cache write are one kernel between the q|k|v product
    (float32 result) and the attention kernel; softmax, cap and sink are float32 inside it."""

    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, dk: int, dv: int,
                 position: PositionEncoding, scale: Optional[float] = None, window: int = 0, softcap: float = 0.0,
                 sink: bool = False, bias: bool = False, proj_norm: bool = False, head_norm: bool = False,
                 norm_eps: float = 1e-6, value_mix: Optional[str] = None, mix_key: str = "v_first",
                 rotate_values: bool = False, keep_first: int = 0) -> None:
        super().__init__()
        if num_kv_heads < 1 or num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        if value_mix not in (None, "source", "mix"):
            raise ValueError(f"attention: unknown value_mix {value_mix!r}")
        if getattr(position, "rotary_dim", 0) > dk:
            raise ValueError("attention_general: the rotation covers at most the head's own size")
        if rotate_values and (dv % 2 or not hasattr(position, "theta")):
            raise ValueError("attention_general: rotated values need an even value size and a rotary position encoding")
        self.hidden, self.nh, self.nkv, self.dk, self.dv = hidden, num_heads, num_kv_heads, dk, dv
        self.hd = padded_head_dim(max(dk, dv))
        self.window, self.softcap = int(window or 0), float(softcap or 0.0)
        self.keep_first = int(keep_first or 0) if self.window > 0 else 0
        self.rotate_values = bool(rotate_values)
        self._v_inv_freq = None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(dk)
        self.has_sink, self.has_bias, self.proj_norm, self.head_norm = bool(sink), bool(bias), bool(proj_norm), bool(head_norm)
        self.norm_eps, self.value_mix, self.mix_key = float(norm_eps), value_mix, mix_key
        self.position = self.add_child("position", position)
        nq, nk, nv = num_heads * dk, num_kv_heads * dk, num_kv_heads * dv
        self.qkv = self.add_child("qkv", Linear(hidden, nq + nk + nv, hidden ** -0.5))
        self.o = self.add_child("o", Linear(num_heads * dv, hidden, (num_heads * dv) ** -0.5))
        if self.has_bias:
            self.declare("bias", (nq + nk + nv,), ("normal", 0.1), "vector")
        if self.proj_norm:
            self.declare("q_norm", (nq,), ("ones_jitter", 0.1), "vector")
            self.declare("k_norm", (nk,), ("ones_jitter", 0.1), "vector")
        if self.has_sink:
            self.declare("sink", (num_heads,), ("normal", 1.0), "vector")
        if value_mix is not None:
            self.declare("vmix", (), ("normal", 0.3), "vector")       # read by "mix" layers only
        self._f32 = {}
        self._o_weight = None

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(self.nkv, self.hd, 0 if self.keep_first > 0 else self.window)

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        self._f32 = {n: self.param(n).to(device=device, dtype=torch.float32).reshape(-1).contiguous()
                     for n in self.param_specs()}
        if self.rotate_values:
            m = torch.arange(self.dv // 2, dtype=torch.float64)
            self._v_inv_freq = (1.0 / torch.pow(torch.tensor(self.position.theta, dtype=torch.float64),
                                                2.0 * m / self.dv)).to(torch.float32).to(device)
        w = self.o.param("weight")
        if self.hd != self.dv:                              # zero columns where the attention output is padding
            wide = torch.zeros((self.hidden, self.nh, self.hd), dtype=w.dtype, device=w.device)
            wide[:, :, :self.dv] = w.view(self.hidden, self.nh, self.dv)
            w = wide.view(self.hidden, self.nh * self.hd)
        self._o_weight = w

    def forward(self, h: torch.Tensor, ctx: StepContext, site: SiteCache) -> torch.Tensor:
        g = ctx.groups[site.group]
        pos, f = self.position, self._f32
        T = h.shape[0]
        proj = self.qkv.forward(h, ctx, out_dtype=torch.float32)
        keep = first = None
        if self.value_mix == "source":
            keep = ctx.shared[self.mix_key] = torch.empty((T, self.nkv * self.dv), dtype=torch.float32, device=h.device)
        elif self.value_mix == "mix":
            first = ctx.shared[self.mix_key]
        q = torch.empty((T, self.nh * self.hd), dtype=h.dtype, device=h.device)
        K.attn_prepare(proj, f.get("bias"), f.get("q_norm"), f.get("k_norm"), ctx.positions, pos.inv_freq,
                       pos.rotary_dim if pos.inv_freq is not None else 0, self.head_norm, self.norm_eps, keep, first,
                       f["vmix"] if first is not None else None, g.slot_mapping if site.writes else None, q, site.k, site.v,
                       self.nh, self.nkv, self.dk, self.dv, bool(getattr(pos, "interleaved", False)), self._v_inv_freq)
        out = torch.empty((T, self.nh * self.hd), dtype=h.dtype, device=h.device)
        K.paged_attention(q, out, site.k, site.v, g.block_tables, ctx, self.nh, self.nkv, self.hd, self.scale,
                          self.window, self.softcap, f.get("sink"), self.keep_first)
        if self.rotate_values:
            K.rotate_heads(out, ctx.positions, self._v_inv_freq, self.nh, self.hd, bool(getattr(pos, "interleaved", False)), -1.0)
        return matmul_nt(out, self._o_weight, torch.float32, ctx.options)


@MIXERS.register("differential_attention")
class DifferentialAttention(Mixer):
    """Grouped-query attention whose every head forms TWO softmax maps over the same values and subtracts them:

        q = W_q h + b_q  [heads x 2 x dk],   k = W_k h + b_k  [kv_heads x 2 x dk],   v = W_v h + b_v  [kv_heads x dv]
        a_m = softmax(scale * rot(q_m) . rot(k_m)) v        for the maps m = 1, 2 (causal; the rotation covers the first
                                                            ``position.rotary_dim`` elements of each map)
        lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff     (one number for the layer)
        o = (a_1 - lambda a_2) / sqrt(mean(o^2) + eps) * (1 - diff)     per head over its dv values, no weight
        y = W_o concat_heads( sigmoid(w_g,h . h) * o_h ) + b_o           (one gate number per head)

    A key head is cached with its two maps side by side ([k_1 | k_2], 2 dk elements) next to one value head; the
    attention kernels run 2 x heads query heads, each a padded head that holds one map at its own place and zeros at
    the other's, so a query meets only its own map of the key and both maps share the value pages.  Cache head size:
    ``padded_head_dim(max(2 dk, dv))``.  One product gives q | k | v | gate logits (float32 result); bias, rotation
    and the page write are one kernel, the combination of the maps another.  ``out_bias`` is the output product's
    bias; a block that adds it itself sets ``defer_bias``."""

    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, dk: int, dv: int, position: PositionEncoding,
                 diff: float, scale: Optional[float] = None, norm_eps: float = 1e-6, bias: bool = True, gate: bool = True,
                 window: int = 0) -> None:
        super().__init__()
        if num_kv_heads < 1 or num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        if getattr(position, "rotary_dim", 0) > dk:
            raise ValueError("differential_attention: the rotation covers at most one map's size")
        self.hidden, self.nh, self.nkv, self.dk, self.dv = hidden, num_heads, num_kv_heads, dk, dv
        self.hd = padded_head_dim(max(2 * dk, dv))
        self.diff, self.norm_eps, self.window = float(diff), float(norm_eps), int(window or 0)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(dk)
        self.has_bias, self.has_gate = bool(bias), bool(gate)
        self.position = self.add_child("position", position)
        self.nq, self.nk, self.nv = num_heads * 2 * dk, num_kv_heads * 2 * dk, num_kv_heads * dv
        self.qkvg = self.add_child("qkvg", Linear(hidden, self.nq + self.nk + self.nv + (num_heads if gate else 0), hidden ** -0.5))
        self.o = self.add_child("o", Linear(num_heads * dv, hidden, (num_heads * dv) ** -0.5))
        if self.has_bias:
            self.declare("bias", (self.nq + self.nk + self.nv,), ("normal", 0.1), "vector")
            self.declare("o_bias", (hidden,), ("normal", 0.1), "vector")
        for n in ("lq1", "lk1", "lq2", "lk2"):
            self.declare(n, (dk,), ("normal", 0.1), "vector")
        self.defer_bias = False
        self.out_bias: Optional[torch.Tensor] = None
        self._bias = self._lambda = None

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(self.nkv, self.hd, self.window)

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        f = {n: self.param(n).to(device=device, dtype=torch.float32).reshape(-1).contiguous() for n in self.param_specs()}
        self._lambda = (torch.exp((f["lq1"] * f["lk1"]).sum()) - torch.exp((f["lq2"] * f["lk2"]).sum()) + self.diff).reshape(1).contiguous()
        if self.has_bias:
            self._bias, self.out_bias = f["bias"], f["o_bias"]

    def forward(self, h: torch.Tensor, ctx: StepContext, site: SiteCache) -> torch.Tensor:
        g = ctx.groups[site.group]
        pos = self.position
        T, H = h.shape[0], self.nh
        proj = self.qkvg.forward(h, ctx, out_dtype=torch.float32)
        q = torch.empty((T, 2 * H * self.hd), dtype=h.dtype, device=h.device)
        K.attn_prepare(proj, self._bias, None, None, ctx.positions, pos.inv_freq,
                       pos.rotary_dim if pos.inv_freq is not None else 0, False, self.norm_eps, None, None, None,
                       g.slot_mapping if site.writes else None, q, site.k, site.v, H, self.nkv, self.dk, self.dv,
                       bool(getattr(pos, "interleaved", False)), None, maps=2)
        maps = torch.empty((T, 2 * H, self.hd), dtype=h.dtype, device=h.device)
        K.paged_attention(q, maps.view(T, 2 * H * self.hd), site.k, site.v, g.block_tables, ctx, 2 * H, self.nkv, self.hd,
                          self.scale, self.window)
        out = torch.empty((T, H * self.dv), dtype=h.dtype, device=h.device)
        K.diff_combine(maps, proj[:, self.nq + self.nk + self.nv:] if self.has_gate else None, self._lambda, out, H, self.dv,
                       self.norm_eps, 1.0 - self.diff)
        y = self.o.forward(out, ctx, out_dtype=torch.float32)
        if self.out_bias is not None and not self.defer_bias:
            K.add_bias_rows(y, self.out_bias)
        return y
