"""Attention over a cached latent: per position one normalised vector c [rank] is kept, and every
head's keys and values are linear in it, k = W_uk c and v = W_uv c.  No position encoding.

    q = W_q h;   c = w * (W_dkv h) / rms(W_dkv h);   score_ij = scale * q_i . k_j  (j <= i);
    out = W_o concat_heads( softmax(score) v )

Only c is cached, in pages laid out like a key pool with ONE shared head of ``rank`` elements and
no value pool.  The products with W_uk and W_uv are moved across the softmax, which changes
nothing in exact arithmetic: score = (W_uk^T q) . c and sum_j p_j W_uv c_j = W_uv (sum_j p_j c_j).
So every head's query is mapped into the latent space, the engine's paged attention kernels run
with all heads sharing the latent pages as keys AND values (prefill and decode alike, portions
reading earlier portions' latents from the pages), and the head outputs are mapped back by W_uv.
A site built with ``own_latent=False`` has no W_dkv: the run order points it at an earlier site's
pages (``LayerCall.cache_of``), which it reads with its own W_uk, W_uv and queries.
"""
from __future__ import annotations

import torch

from ..kernels import library as K
from .base import CacheSpec, MIXERS, Mixer, SiteCache, StepContext
from .linear import Linear

BMM_MIN_ROWS = 64       # from here on the library's batched product does the per-head maps of bfloat16 rows


def per_head_product(x: torch.Tensor, w: torch.Tensor, ctx: StepContext, out: torch.Tensor = None) -> torch.Tensor:
    """x [M, B, K] (a view; K dense), w [B, N, K] -> [M, B * N]: y[m, b] = w[b] x[m, b].  ``out`` [M, B, N] (a view
    with dense last dimension) receives the result instead of a new tensor and is returned as it is."""
    M, B, _ = x.shape
    N = w.shape[1]
    y = torch.empty((M, B, N), dtype=x.dtype, device=x.device) if out is None else out
    if x.dtype == torch.bfloat16 and M >= BMM_MIN_ROWS and ctx.options.get("gemm", "auto") in ("auto", "library"):
        torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=y.transpose(0, 1))
        K.profile_mark("library_gemm")
    else:
        K.gemm_plain_batched(x, w, y)
    return y.view(M, B * N) if out is None else out


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, hidden: int, heads: int, dk: int, dv: int, rank: int, scale: float, norm_eps: float,
                 own_latent: bool = True) -> None:
        super().__init__()
        self.hidden, self.heads, self.dk, self.dv, self.rank = hidden, heads, dk, dv, rank
        self.scale, self.norm_eps, self.own_latent = float(scale), float(norm_eps), bool(own_latent)
        std = hidden ** -0.5
        # one product for q | (latent before its norm)
        self.q_dkv = self.add_child("q_dkv", Linear(hidden, heads * dk + (rank if own_latent else 0), std))
        self.uk = self.add_child("uk", Linear(rank, heads * dk, rank ** -0.5))
        self.uv = self.add_child("uv", Linear(rank, heads * dv, rank ** -0.5))
        self.o = self.add_child("o", Linear(heads * dv, hidden, (heads * dv) ** -0.5))
        if own_latent:
            self.declare("latent_norm", (rank,), ("ones",), "vector")
        self._uk_t = self._uv = self._norm = None

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(1, self.rank, 0, values=False)

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        H, R = self.heads, self.rank
        # W_uk [H*dk, R] as H maps from a head's query to the latent space: [H, R, dk]
        self._uk_t = self.uk.param("weight").view(H, self.dk, R).transpose(1, 2).contiguous()
        self._uv = self.uv.param("weight").view(H, self.dv, R)
        if self.own_latent:
            self._norm = self.param("latent_norm").to(device=device, dtype=torch.float32).contiguous()

    def forward(self, h: torch.Tensor, ctx: StepContext, site: SiteCache) -> torch.Tensor:
        g = ctx.groups[site.group]
        M, H, R = h.shape[0], self.heads, self.rank
        proj = self.q_dkv.forward(h, ctx)
        if self.own_latent:
            if not site.writes:
                raise RuntimeError("latent_attention: a site with a latent of its own must own its pages")
            K.latent_norm_cache(proj[:, H * self.dk:], self._norm, g.slot_mapping, site.k, self.norm_eps)
        q_lat = per_head_product(proj[:, :H * self.dk].unflatten(1, (H, self.dk)), self._uk_t.to(proj.dtype), ctx)
        out_lat = torch.empty((M, H * R), dtype=h.dtype, device=h.device)
        pages = site.k
        if (h.dtype == torch.bfloat16 and ctx.options.get("attention", "auto") != "plain"
                and K.fast_attention_supported(H, 1, R, pages.shape[2]) and (H * R) % 8 == 0):
            K.paged_attention(q_lat, out_lat, pages, pages, g.block_tables, ctx, H, 1, R, self.scale, 0)
        else:
            K.attention_plain(q_lat, out_lat, pages, pages, g.block_tables, ctx.row_seq, ctx.positions, H, 1, R,
                              self.scale, 0)
        heads_out = per_head_product(out_lat.view(M, H, R), self._uv.to(out_lat.dtype), ctx)
        return self.o.forward(heads_out, ctx, out_dtype=torch.float32)


@MIXERS.register("latent_rope_attention")
class LatentRopeAttention(Mixer):
    """Attention over a cached latent with a rotated key part beside it and queries that go through a latent
    of their own:

        c_q = w_q * (W_dq h) / rms(W_dq h);      q = W_uq c_q, per head [dn unrotated | dr rotated]
        W_dkv h = [c_raw: rank | k_r: dr];       c = w_c * c_raw / rms(c_raw);   k_r: one part shared by all heads
        score_ij = scale * (q_n,i . (W_uk c_j) + rot(q_r,i) . rot(k_r,j))   (j <= i),   v_j = W_uv c_j
        out = W_o concat_heads( softmax(score) v )

    rot turns the first ``position.rotary_dim`` elements of the dr-part by the position.  Only [c | rot(k_r)] is
    cached: pages laid out like a key pool with ONE shared head of ``padded_head_dim(rank + dr)`` elements (zeros
    behind) and no value pool.  As in ``latent_attention`` the maps W_uk and W_uv move across the softmax: every
    head's query becomes [W_uk^T q_n | rot(q_r) | 0], the engine's paged attention kernels run with all heads
    sharing the pages as keys AND values, and W_uv maps the first ``rank`` elements of a head's output back.
    Norms, angles and the turn are float32 (the dq|dkv and uq products return float32).

    Options: ``q_rank`` = 0: the queries have no latent, q = W_q h comes out of the first product (q | dkv);
    ``window`` > 0: position i sees j with 0 <= i - j < window (the pages behind the window are given back);
    ``sink``: a learned number per head whose exponential joins the softmax's denominator; ``gate``: the
    concatenated heads are multiplied element by element with sigmoid(W_g h), W_g's rows being the last of the
    first product."""

    def __init__(self, hidden: int, heads: int, dn: int, dr: int, dv: int, rank: int, q_rank: int, scale: float,
                 norm_eps: float, position, window: int = 0, sink: bool = False, gate: bool = False) -> None:
        super().__init__()
        from .attention import padded_head_dim
        if getattr(position, "rotary_dim", 0) > dr:
            raise ValueError("latent_rope_attention: the rotation covers at most the rotated part")
        self.hidden, self.heads, self.dn, self.dr, self.dv, self.rank, self.q_rank = hidden, heads, dn, dr, dv, rank, int(q_rank or 0)
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.window, self.has_sink, self.has_gate = int(window or 0), bool(sink), bool(gate)
        self.hd = padded_head_dim(rank + dr)
        self.position = self.add_child("position", position)
        std = hidden ** -0.5
        self.nq = heads * (dn + dr)
        # one product: (dq, or q itself when the queries have no latent) | dkv | gate logits
        self.n_first = self.q_rank if self.q_rank else self.nq
        self.dq_dkv = self.add_child("dq_dkv", Linear(hidden, self.n_first + rank + dr + (heads * dv if gate else 0), std))
        if self.q_rank:
            self.uq = self.add_child("uq", Linear(self.q_rank, self.nq, self.q_rank ** -0.5))
            self.declare("q_norm", (self.q_rank,), ("ones_jitter", 0.1), "vector")
        self.uk = self.add_child("uk", Linear(rank, heads * dn, rank ** -0.5))
        self.uv = self.add_child("uv", Linear(rank, heads * dv, rank ** -0.5))
        self.o = self.add_child("o", Linear(heads * dv, hidden, (heads * dv) ** -0.5))
        self.declare("latent_norm", (rank,), ("ones_jitter", 0.1), "vector")
        if self.has_sink:
            self.declare("sink", (heads,), ("normal", 1.0), "vector")
        self._uk_t = self._uv = None
        self._f32 = {}

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(1, self.hd, self.window, values=False)

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        H, R = self.heads, self.rank
        self._uk_t = self.uk.param("weight").view(H, self.dn, R).transpose(1, 2).contiguous()     # [H, R, dn]
        self._uv = self.uv.param("weight").view(H, self.dv, R)
        self._f32 = {n: self.param(n).to(device=device, dtype=torch.float32).contiguous() for n in self.param_specs()}

    def forward(self, h: torch.Tensor, ctx: StepContext, site: SiteCache) -> torch.Tensor:
        if not site.writes:
            raise RuntimeError("latent_rope_attention: the call site must own its pages")
        g = ctx.groups[site.group]
        pos = self.position
        M, H, R, HD = h.shape[0], self.heads, self.rank, self.hd
        proj = self.dq_dkv.forward(h, ctx, out_dtype=torch.float32)
        if self.q_rank:
            cq = torch.empty((M, self.q_rank), dtype=h.dtype, device=h.device)
            K.latent_rope_cache(proj, self._f32["q_norm"], self._f32["latent_norm"], ctx.positions, pos.inv_freq, pos.interleaved,
                                g.slot_mapping, cq, site.k, self.q_rank, R, self.dr, self.norm_eps)
            q = self.uq.forward(cq, ctx, out_dtype=torch.float32)
        else:
            K.latent_rope_cache(proj[:, self.nq:], None, self._f32["latent_norm"], ctx.positions, pos.inv_freq, pos.interleaved,
                                g.slot_mapping, None, site.k, 0, R, self.dr, self.norm_eps)
            q = proj[:, :self.nq]
        qn = torch.empty((M, H, self.dn), dtype=h.dtype, device=h.device)
        qrow = torch.empty((M, H, HD), dtype=h.dtype, device=h.device)
        K.latent_q_rope(q, ctx.positions, pos.inv_freq, pos.interleaved, qn, qrow, H, self.dn, self.dr, R)
        per_head_product(qn, self._uk_t.to(qn.dtype), ctx, out=qrow[:, :, :R])
        out_lat = torch.empty((M, H, HD), dtype=h.dtype, device=h.device)
        pages = site.k
        K.paged_attention(qrow.view(M, H * HD), out_lat.view(M, H * HD), pages, pages, g.block_tables, ctx, H, 1, HD,
                          self.scale, self.window, 0.0, self._f32.get("sink"))
        heads_out = per_head_product(out_lat[:, :, :R], self._uv.to(out_lat.dtype), ctx)
        if self.has_gate:
            K.gate_mul(heads_out, proj[:, self.n_first + R + self.dr:], heads_out)
        return self.o.forward(heads_out, ctx, out_dtype=torch.float32)
