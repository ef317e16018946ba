"""Token embedding (gather into the float32 residual stream, no scaling:
``src/cuda/kernels.cu:27-32``) and the output head (logits in float32 for the wanted rows only:
``src/model/llama.cpp:126-128``)."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import library as K
from .base import Part, StepContext
from .linear import matmul_nt


class Embedding(Part):
    def __init__(self, vocab: int, hidden: int) -> None:
        super().__init__()
        self.vocab, self.hidden = vocab, hidden
        self.declare("weight", (vocab, hidden), ("normal", 0.02), "table")

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = torch.empty((ctx.rows, self.hidden), dtype=torch.float32, device=ctx.tokens.device)
        K.embed(ctx.tokens, self.param("weight"), x)
        return x


class ScaledEmbedding(Part):
    """x = table[token] * scale into the float32 residual stream.  With ``keep_as`` the same rows are also left
    in ``ctx.shared[keep_as]`` (float32) for parts that read the embedding's output later in the step."""

    def __init__(self, vocab: int, hidden: int, scale: float = 1.0, keep_as: Optional[str] = None) -> None:
        super().__init__()
        self.vocab, self.hidden, self.scale, self.keep_as = vocab, hidden, float(scale), keep_as
        self.declare("weight", (vocab, hidden), ("normal", 0.02), "table")

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = torch.empty((ctx.rows, self.hidden), dtype=torch.float32, device=ctx.tokens.device)
        keep = None
        if self.keep_as:
            keep = ctx.shared[self.keep_as] = torch.empty_like(x)
        K.embed_scaled(ctx.tokens, self.param("weight"), x, keep, self.scale)
        return x


class SummedEmbedding(Part):
    """A sum of tables into the float32 residual stream: the token's row; optionally the row of a
    hashed table for the pair (previous token, token), row ``(prev * mul_prev + token * mul_cur) mod
    buckets`` and the extra last row ``buckets`` for a request's first token; optionally a learned
    row per position (not scaled).  The previous token comes with the batch (the request keeps its
    tokens), so it survives portions, batching and eviction like the tokens themselves."""

    def __init__(self, vocab: int, hidden: int, buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0,
                 max_positions: int = 0) -> None:
        super().__init__()
        self.vocab, self.hidden = vocab, hidden
        self.buckets, self.mul_prev, self.mul_cur, self.max_positions = int(buckets), int(mul_prev), int(mul_cur), int(max_positions)
        self.declare("weight", (vocab, hidden), ("normal", 0.02), "table")
        if self.buckets:
            self.declare("pair", (self.buckets + 1, hidden), ("normal", 0.02), "table")
        if self.max_positions:
            self.declare("place", (self.max_positions, hidden), ("normal", 0.02), "table")

    def forward(self, ctx: StepContext) -> torch.Tensor:
        table = self.param("weight")
        x = torch.empty((ctx.rows, self.hidden), dtype=torch.float32, device=ctx.tokens.device)
        h = None
        if ctx.dtype != torch.float32 and table.dtype == ctx.dtype:
            h = ctx.h_stream = torch.empty((ctx.rows, self.hidden), dtype=ctx.dtype, device=x.device)
        K.embed_sum(ctx.tokens, ctx.prev_tokens, ctx.positions, table, self.param("pair") if self.buckets else None,
                    self.param("place") if self.max_positions else None, x, h, self.buckets, self.mul_prev, self.mul_cur)
        return x


class LMHead(Part):
    """logits = h W^T in float32.  ``weight`` may alias the embedding table (tied).  ``softcap`` > 0:
    logits <- cap * tanh(logits / cap)."""

    def __init__(self, hidden: int, vocab: int, softcap: float = 0.0) -> None:
        super().__init__()
        self.vocab, self.hidden, self.softcap = vocab, hidden, float(softcap or 0.0)
        self.declare("weight", (vocab, hidden), ("normal", 0.02), "matrix")

    def forward(self, h: torch.Tensor, ctx: Optional[StepContext] = None) -> torch.Tensor:
        logits = matmul_nt(h, self.param("weight"), torch.float32, ctx.options if ctx else {})
        if self.softcap > 0.0:
            K.softcap_rows(logits, self.softcap)
        return logits
