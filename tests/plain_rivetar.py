"""Rivetar restated plainly: float64 torch on the CPU, whole sequences at once, one function per
mechanism, written from the design's equations and sharing no code with the engine.

A model is (cfg, tensors): ``cfg`` the parsed config.json, ``tensors`` name -> float64 tensor.
``forward(cfg, tensors, tokens)`` returns the logits of every position; ``trace`` additionally the
residual stream after every layer run.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

F = torch.float64


def rms_div(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """x / rms(x) * (1 + w): the weight is stored as its distance from one."""
    return rms_div(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms_div(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, base: float, dims: int, sign: float = 1.0) -> torch.Tensor:
    """x [T, heads, n]: the first ``dims`` elements of every head, pair (2i, 2i+1), turn by
    sign * pos * base^(-2i/dims); the rest pass."""
    out = x.clone()
    half = dims // 2
    i = torch.arange(half, dtype=F)
    ang = sign * pos.to(F)[:, None] * base ** (-2.0 * i / dims)[None, :]          # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def visible(T: int, window: int = 0, keep_first: int = 0) -> torch.Tensor:
    """[T, T] bool: row i sees column j when j <= i and (no window, or i - j < window, or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window > 0:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def softmax_with_sink(scores: torch.Tensor, mask: torch.Tensor, sink=None) -> torch.Tensor:
    """scores [H, T, T]; returns weights over the visible keys; with ``sink`` [H] the denominator
    also holds exp(sink_h)."""
    s = scores.masked_fill(~mask[None], float("-inf"))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return e / den


def mixer_latent_attention(h, m, w: Dict[str, torch.Tensor], eps: float):
    T = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = norm_plain(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(T, H, dn + dr)
    q_n, q_r = q[..., :dn], q[..., dn:]
    dkv = h @ w["dkv"].T
    c = norm_plain(dkv[:, :R], w["dkv.norm"], eps)
    k_r = dkv[:, R:].view(T, 1, dr)
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q_r = rotate_pairs(q_r, pos, base, dims)
    k_r = rotate_pairs(k_r, pos, base, dims)
    k_n = (c @ w["uk"].T).view(T, H, dn)
    v = (c @ w["uv"].T).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_n, k_n) + torch.einsum("ihd,jd->hij", q_r, k_r[:, 0])) * m["scale"]
    p = softmax_with_sink(scores, visible(T))
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv)
    return o @ w["o"].T


def mixer_attention(h, m, w, eps: float):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w["q"].T).view(T, H, dk)
    k = (h @ w["k"].T).view(T, G, dk)
    v = (h @ w["v"].T).view(T, G, dv)
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q = rotate_pairs(q, pos, base, dims)
    k = rotate_pairs(k, pos, base, dims)
    v = rotate_pairs(v, pos, base, dv)                      # values turn by their own position, over all of vdim
    rep = H // G
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    mask = m.get("mask") or {}
    p = softmax_with_sink(scores, visible(T, mask.get("size", 0), mask.get("keep_first", 0)), w["sink"])
    o = torch.einsum("hij,jhd->ihd", p, v)
    o = rotate_pairs(o, pos, base, dv, sign=-1.0)           # and the sum turns back by the reader's position
    return o.reshape(T, H * dv) @ w["o"].T


def mixer_gla(h, m, w, eps: float):
    T = h.shape[0]
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    q = (h @ w["q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w["k"].T).view(T, H, dk)
    v = (h @ w["v"].T).view(T, H, dv)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / tau).view(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=F)
    o = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = norm_plain(o, w["norm"], eps).reshape(T, H * dv)
    g = h @ w["g"].T
    return (o * (g * torch.sigmoid(g))) @ w["o"].T


def poly_norm(z, coef, eps):
    a, b, c, e = [float(t) for t in coef]
    return a * rms_div(z, eps) + b * rms_div(z ** 2, eps) + c * rms_div(z ** 3, eps) + e


def feed_forward(h, w, eps):
    return poly_norm(h @ w["up"].T, w["act"], eps) @ w["down"].T


MIXERS = {"latent_attention": mixer_latent_attention, "attention": mixer_attention, "gla": mixer_gla}


def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def layer(x, cfg, tensors, i: int):
    eps = cfg["norm"]["eps"]
    L = cfg["layers"][i]
    p = f"l{i}."
    y = MIXERS[L["type"]](norm_around_zero(x, tensors[p + "norm1"], eps), L["mixer"], sub(tensors, p + "mix."), eps)
    x = x + norm_around_zero(y, tensors[p + "norm1b"], eps)
    if L.get("mlp") is not None:
        y = feed_forward(norm_around_zero(x, tensors[p + "norm2"], eps), sub(tensors, p + "mlp."), eps)
        x = x + norm_around_zero(y, tensors[p + "norm2b"], eps)
    return x


def run_order(cfg) -> List[tuple]:
    """(layer, pass number or None, first of its pass)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    out = [(i, None, False) for i in range(a)]
    for t in range(times):
        out += [(i, t, i == a) for i in range(a, b)]
    out += [(i, None, False) for i in range(b, n)]
    return out


def trace(cfg, tensors, tokens):
    tensors = {k: v.to(F) for k, v in tensors.items()}
    x0 = tensors["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    x = x0
    streams = []
    for i, t, first in run_order(cfg):
        if first:
            x = torch.cat([x, x0], dim=-1) @ tensors["loop.in"].T + tensors["loop.step"][t]
        x = layer(x, cfg, tensors, i)
        streams.append(x)
    hn = norm_around_zero(x, tensors["final.norm"], cfg["norm"]["eps"])
    logits = hn @ tensors["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits, streams


def forward(cfg, tensors, tokens):
    return trace(cfg, tensors, tokens)[0]
