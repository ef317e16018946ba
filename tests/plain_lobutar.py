"""Lobutar restated plainly: float64 torch on the CPU, whole sequences at once, one function per
mechanism, written from the design's equations and sharing no code with the engine.

A model is (cfg, tensors): ``cfg`` the parsed config.json, ``tensors`` name -> float64 tensor.
``forward(cfg, tensors, tokens)`` returns the logits of every position; ``trace`` additionally the
sum of the residual streams after every layer run.
"""
from __future__ import annotations

from typing import Dict, List

import torch

F = torch.float64


def rms_div(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_weighted(x, w, eps):
    return rms_div(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, ..., n]: the first ``dims`` elements of the last axis, pairs (2i, 2i+1), turn by
    pos * base^(-2i/dims); the rest pass."""
    out = x.clone()
    if dims <= 0:
        return out
    i = torch.arange(dims // 2, dtype=F)
    ang = pos.to(F)[:, None] * base ** (-2.0 * i / dims)[None, :]                 # [T, dims/2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def visible(T: int, window: int = 0) -> torch.Tensor:
    """[T, T] bool: row i sees column j when j <= i and (no window or i - j < window)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window > 0:
        ok = ok & (i - j < window)
    return ok


def softmax_visible(scores: torch.Tensor, mask: torch.Tensor, sink=None) -> torch.Tensor:
    """scores [H, T, T]; weights over the visible keys.  With ``sink`` [H] the denominator also holds
    exp(sink_h), which has no key and no value."""
    s = scores.masked_fill(~mask[None], float("-inf"))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return e / den


def differential_lambda(w: Dict[str, torch.Tensor], diff: float) -> torch.Tensor:
    return torch.exp((w["lq1"] * w["lk1"]).sum()) - torch.exp((w["lq2"] * w["lk2"]).sum()) + diff


def mixer_attention(h, m, w: Dict[str, torch.Tensor], eps: float):
    """Differential attention: two softmax maps per head over the same values, subtracted."""
    T = h.shape[0]
    H, G, dk, dv, diff = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["diff"]
    pos = torch.arange(T)
    q = (h @ w["q"].T + w["q.b"]).view(T, H, 2, dk)
    k = (h @ w["k"].T + w["k.b"]).view(T, G, 2, dk)
    v = (h @ w["v"].T + w["v.b"]).view(T, G, dv)
    if m.get("rot"):
        q = rotate_pairs(q, pos, m["rot"]["base"], m["rot"]["dims"])
        k = rotate_pairs(k, pos, m["rot"]["base"], m["rot"]["dims"])
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)                      # head h uses key/value head h // rep
    vv = v.repeat_interleave(rep, dim=1)
    mask = visible(T)
    maps = []
    for j in range(2):
        s = torch.einsum("ihd,jhd->hij", q[:, :, j], kk[:, :, j]) * m["scale"]
        p = softmax_visible(s, mask)
        maps.append(torch.einsum("hij,jhd->ihd", p, vv))
    lam = differential_lambda(w, diff)
    o = maps[0] - lam * maps[1]
    o = rms_div(o, eps) * (1.0 - diff)
    gate = torch.sigmoid(h @ w["g"].T)                        # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * dv) @ w["o"].T + w["o.b"]


def mixer_latent_attention(h, m, w: Dict[str, torch.Tensor], eps: float):
    T = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ w["q"].T).view(T, H, dn + dr)
    q_n, q_r = q[..., :dn], q[..., dn:]
    dkv = h @ w["dkv"].T
    c = norm_weighted(dkv[:, :R], w["dkv.norm"], eps)
    k_r = dkv[:, R:]                                          # [T, dr], one part for all heads
    q_r = rotate_pairs(q_r, pos, m["rot"]["base"], m["rot"]["dims"])
    k_r = rotate_pairs(k_r, pos, m["rot"]["base"], m["rot"]["dims"])
    k_n = (c @ w["uk"].T).view(T, H, dn)
    v = (c @ w["uv"].T).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q_n, k_n) + torch.einsum("ihd,jd->hij", q_r, k_r)) * m["scale"]
    window = (m.get("mask") or {}).get("size", 0)
    p = softmax_visible(s, visible(T, window), w["sink"])
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def gated_ff(h, w, prefix: str):
    return (silu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def route(h, w, r) -> (torch.Tensor, torch.Tensor):
    """Returns (chosen experts [T, top], their weights [T, top])."""
    E, top = r["experts"], r["top"]
    z = h @ w["router"].T
    s = torch.sigmoid(z)
    choice = s + w["correction"]
    groups = r.get("groups")
    if groups and groups["count"] > 1:
        n, keep = groups["count"], groups["keep"]
        per = E // n
        g = choice.view(-1, n, per)
        gscore = g.topk(min(2, per), dim=-1).values.sum(-1)   # a group's two largest choice scores
        best = gscore.topk(keep, dim=-1).indices
        allowed = torch.zeros(h.shape[0], n, dtype=torch.bool)
        allowed.scatter_(1, best, True)
        choice = choice.masked_fill(~allowed[:, :, None].expand(-1, -1, per).reshape(-1, E), float("-inf"))
    idx = choice.topk(top, dim=-1).indices
    return idx, s.gather(1, idx) * r.get("scale", 1.0)


def feed_forward(h, mlp, w: Dict[str, torch.Tensor]):
    if mlp["kind"] == "dense":
        return gated_ff(h, w, "")
    idx, wt = route(h, w, mlp["router"])
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(idx.shape[1]):
            e = int(idx[t, k])
            y[t] += wt[t, k] * gated_ff(h[t:t + 1], w, f"e{e}.")[0]
    if mlp.get("shared"):
        y = y + gated_ff(h, w, "shared.")
    return y


def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def hyper_read(xs: torch.Tensor, hc: Dict[str, torch.Tensor]) -> torch.Tensor:
    """xs [S, T, D] -> the sublayer's input sum_s in[s] xs[s]."""
    return torch.einsum("s,std->td", hc["in"], xs)


def hyper_write(xs: torch.Tensor, y: torch.Tensor, hc: Dict[str, torch.Tensor]) -> torch.Tensor:
    """new[t] = sum_s mix[s, t] xs[s] + out[t] y, all streams from the old ones."""
    return torch.einsum("sr,std->rtd", hc["mix"], xs) + hc["out"][:, None, None] * y[None]


def layer(xs, spec, tensors, i: int, eps: float):
    """One layer run on the streams xs [S, T, D]; ``i`` is the layer whose tensors are used."""
    p = f"l{i}."
    mix = {"attention": mixer_attention, "latent_attention": mixer_latent_attention}[spec["type"]]
    u = hyper_read(xs, sub(tensors, p + "hc1."))
    y = mix(norm_weighted(u, tensors[p + "norm1"], eps), spec["mixer"], sub(tensors, p + "mix."), eps)
    xs = hyper_write(xs, y, sub(tensors, p + "hc1."))
    if spec.get("mlp") is not None:
        u = hyper_read(xs, sub(tensors, p + "hc2."))
        y = feed_forward(norm_weighted(u, tensors[p + "norm2"], eps), spec["mlp"], sub(tensors, p + "mlp."))
        xs = hyper_write(xs, y, sub(tensors, p + "hc2."))
    return xs


def trace(cfg, tensors: Dict[str, torch.Tensor], tokens: List[int]):
    eps = cfg["norm"]["eps"]
    x0 = tensors["embed"][torch.tensor(tokens)]
    xs = x0[None].repeat(cfg["streams"], 1, 1)
    after = []
    for i, spec in enumerate(cfg["layers"]):
        xs = layer(xs, spec, tensors, spec.get("weights_of", i), eps)
        after.append(xs.sum(0))
    x = xs.sum(0)
    logits = norm_weighted(x, tensors["final.norm"], eps) @ tensors["head"].T
    return logits, after


def forward(cfg, tensors, tokens):
    return trace(cfg, tensors, tokens)[0]
