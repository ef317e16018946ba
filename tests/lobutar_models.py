"""Small Lobutar configurations for the tests, their model folders and the plain implementation's logits.
The configurations differ from each other in every size and constant, put the layer kinds in different orders,
and avoid values that would hide a mix-up: as many KV heads as heads, a value size equal to twice the key size,
a rotation over a whole map, one stream, groups of which all are kept, a router scale of 1.

lob-a: three streams; differential attention on 2 KV heads with a partial rotation and a dense feed-forward, run a
       second time with the same weights two layers later; a latent layer with a window of 37 and grouped experts
       with a shared one, also run twice; a latent layer without a window and without a feed-forward.
lob-b: two streams; sizes that the tensor-core kernels take (a cached latent row of 112 + 16 = 128 on pages of 32,
       key pairs of 2 x 32 and 2 x 64 elements, experts of 64); one KV head; experts without groups and without a
       shared expert whose size takes the plain expert kernels.
lob-c: ONE stream; a mixer-only first layer; a window of 9 on pages of 8; one expert per token out of four in
       groups that are all kept; a router without a scale.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch

import plain_lobutar as P


def attn(heads, kv, dim, vdim, diff, scale, rot):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "diff": diff, "scale": scale}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, window=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    if window:
        m["mask"] = {"size": window}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None, scale=None, shared=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        r["scale"] = scale
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        m["shared"] = {"ff": shared}
    return m


_A0 = {"type": "attention", "mixer": attn(4, 2, 12, 20, 0.35, 0.3, (10000.0, 8)), "mlp": dense(100)}
_A1 = {"type": "latent_attention", "mixer": latent(3, 16, 8, 20, 40, 0.2, 5000.0, 37), "mlp": moe(8, 2, 24, (4, 2), 1.5, 40)}
_B0 = {"type": "latent_attention", "mixer": latent(4, 32, 16, 48, 112, 0.15, 1000000.0, 70), "mlp": moe(16, 4, 64, (2, 1), 2.0, 96)}
_C1 = {"type": "latent_attention", "mixer": latent(5, 6, 6, 10, 12, 0.45, 20.0, 9), "mlp": moe(4, 1, 10, (2, 2))}

CONFIGS = {
    "lob-a": dict(seed=51, block_size=16, cfg={
        "architecture": "Lobutar", "vocab": 211, "width": 72, "norm": {"eps": 2e-5}, "streams": 3,
        "layers": [_A0, _A1, dict(_A0, weights_of=0),
                   {"type": "latent_attention", "mixer": latent(2, 12, 4, 8, 24, 0.35, 77.0), "mlp": None},
                   dict(_A1, weights_of=1)]}),
    "lob-b": dict(seed=52, block_size=32, cfg={
        "architecture": "Lobutar", "vocab": 150, "width": 128, "norm": {"eps": 1e-6}, "streams": 2,
        "layers": [_B0,
                   {"type": "attention", "mixer": attn(4, 1, 32, 64, 0.8, 0.15, (50000.0, 32)), "mlp": dense(160)},
                   {"type": "attention", "mixer": attn(2, 2, 64, 96, 0.2, 0.1, (777.0, 16)), "mlp": moe(5, 2, 20, None, 0.7)},
                   dict(_B0, weights_of=0)]}),
    "lob-c": dict(seed=53, block_size=8, cfg={
        "architecture": "Lobutar", "vocab": 97, "width": 40, "norm": {"eps": 1e-4}, "streams": 1,
        "layers": [{"type": "attention", "mixer": attn(3, 1, 10, 14, 0.1, 0.35, (50.0, 2)), "mlp": None},
                   _C1, dict(_C1, weights_of=1)]}),
}

TORCH_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def decisive_routers(cfg: dict, w: Dict[str, torch.Tensor], seed: int) -> None:
    """Makes every router's choice a clear one, so that a rounding of the 16-bit path cannot turn it (two experts of
    nearly equal score are no fault of the engine, but they move a position's logits by much).  Every routed layer
    gets residual coordinates of its own, one per expert.  On them the token table holds a permutation of evenly
    spaced codes per token, and no sublayer writes there (the rows of every output matrix and bias are zero), so
    through all layers a stream holds a multiple of the code; the router reads exactly these coordinates.  A row's
    router logits are then a scaled permutation that depends on its token.  The corrections are whole steps of 2
    (more than any difference of two scores): one step count per group where the router has groups, so that the
    corrections alone rank the groups and the scores rank the experts inside them; else a step for some experts,
    which then win over all others.  A router that ignored the corrections would choose other experts."""
    g = torch.Generator().manual_seed(seed)
    at = 0
    for i, layer in enumerate(cfg["layers"]):
        mlp = layer.get("mlp")
        if not mlp or mlp["kind"] != "moe" or layer.get("weights_of") is not None:
            continue
        E = mlp["router"]["experts"]
        cols = slice(at, at + E)
        at += E
        assert at <= cfg["width"]
        codes = torch.stack([torch.randperm(E, generator=g) for _ in range(cfg["vocab"])]).float()
        w["embed"][:, cols] = ((codes - (E - 1) / 2) * (3.0 / E)).to(w["embed"].dtype)
        for name in w:
            if name.endswith((".mix.o", ".mlp.down", ".shared.down")) or (".mlp.e" in name and name.endswith(".down")):
                w[name][cols] = 0
            if name.endswith(".mix.o.b"):
                w[name][cols] = 0
        router = torch.zeros_like(w[f"l{i}.mlp.router"])
        router[:, cols] = 2.0 * torch.eye(E, dtype=router.dtype)
        w[f"l{i}.mlp.router"] = router
        count = (mlp["router"].get("groups") or {}).get("count", 1)
        if count > 1:
            steps = torch.randperm(count, generator=g).repeat_interleave(E // count)
        else:
            steps = torch.randint(0, 2, (E,), generator=g)
        w[f"l{i}.mlp.correction"] = (2.0 * steps).to(w[f"l{i}.mlp.correction"].dtype)
        w[f"l{i}.norm2"][cols] = 1.0


def write_model_from(cfg_dict: dict, seed: int, dtype: str, folder: str, head_scale: float = 40.0, decisive: bool = True) -> str:
    """Random weights through the package's own writer; the token table is scaled up to a spread of 0.5 and the
    output head so that the logits spread over several units."""
    import kvcm
    from safetensors import safe_open
    from safetensors.torch import save_file
    cfg = kvcm.config.config_from_dict(cfg_dict)
    kvcm.write_random_model(folder, cfg, seed, TORCH_DT[dtype])
    path = os.path.join(folder, "model.safetensors")
    w = {}
    with safe_open(path, framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).clone()
    w["head"] = (w["head"].float() * head_scale).to(w["head"].dtype)
    w["embed"] = (w["embed"].float() * 25.0).to(w["embed"].dtype)
    if decisive:
        decisive_routers(cfg_dict, w, seed)
    save_file(w, path, metadata={"format": "pt"})
    return folder


def write_model(name: str, dtype: str, folder: str) -> str:
    c = CONFIGS[name]
    return write_model_from(c["cfg"], c["seed"], dtype, folder)


def read_model(folder: str):
    """(config dict, weights as float64)."""
    from safetensors import safe_open
    cfg = json.load(open(os.path.join(folder, "config.json")))
    w: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).double()
    return cfg, w


def save_weights(folder: str, w: Dict[str, torch.Tensor], dtype: str) -> None:
    from safetensors.torch import save_file
    save_file({n: t.to(TORCH_DT[dtype]).contiguous() for n, t in w.items()}, os.path.join(folder, "model.safetensors"),
              metadata={"format": "pt"})


def plain_logits(folder: str, tokens: List[int]) -> torch.Tensor:
    cfg, w = read_model(folder)
    return P.forward(cfg, w, list(tokens))
