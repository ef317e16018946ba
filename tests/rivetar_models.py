"""Small Rivetar configurations for the tests, their model folders and the plain implementation's logits.
The configurations differ from each other in every size and constant, put the layer kinds in different
orders, and avoid values that would hide a mix-up: key size equal to value size, a rotation over the whole
rotated part, as many KV heads as heads, a window without kept tokens (or kept tokens that never matter),
a loop that starts at the first layer or runs once, scales of 1.

riv-a: a looped span in the middle (layers 1..2, three passes); attention with a window of 37 that keeps 3
       first tokens; a decay rank that is no multiple of 8; latent layers whose rotation covers half of the
       rotated part; a mixer-only attention layer without a window.
riv-b: sizes that the tensor-core kernels take (latent 112 + 16 = one head of 128 on pages of 32; attention heads
       of 64 with a plain window -- and with kept tokens, which takes the other prefill kernel; a state of
       64 x 64); no loop, no cap on the logits.
riv-c: every layer inside the loop (two passes), one gla head, more kept tokens than the window is long,
       one KV head, odd ranks, pages of 8.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch

import plain_rivetar as P


def attn(heads, kv, dim, vdim, scale, rot, window=None, keep=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"base": rot[0], "dims": rot[1]}}
    if window:
        m["mask"] = {"size": window}
        if keep is not None:
            m["mask"]["keep_first"] = keep
    return m


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
            "scale": scale, "rot": {"base": rot[0], "dims": rot[1]}}


def gla(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}


def dense(ff):
    return {"kind": "dense", "ff": ff}


CONFIGS = {
    "riv-a": dict(seed=41, block_size=16, cfg={
        "architecture": "Rivetar", "vocab": 211, "width": 72, "norm": {"eps": 2e-5}, "embedding": {"scale": 2.5},
        "logit_softcap": 20.0, "loop": {"start": 1, "stop": 3, "times": 3},
        "layers": [
            {"type": "attention", "mixer": attn(4, 2, 24, 40, 0.3, (10000.0, 16), 37, 3), "mlp": dense(100)},
            {"type": "gla", "mixer": gla(3, 20, 12, 8.0, 5), "mlp": None},
            {"type": "latent_attention", "mixer": latent(3, 16, 8, 20, 40, 24, 0.2, (5000.0, 4)), "mlp": dense(56)},
            {"type": "attention", "mixer": attn(2, 2, 32, 24, 0.25, (300.0, 32)), "mlp": None},
            {"type": "latent_attention", "mixer": latent(2, 12, 4, 8, 24, 16, 0.35, (77.0, 4)), "mlp": dense(64)},
        ]}),
    "riv-b": dict(seed=42, block_size=32, cfg={
        "architecture": "Rivetar", "vocab": 150, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.5},
        "layers": [
            {"type": "latent_attention", "mixer": latent(4, 32, 16, 48, 112, 64, 0.15, (1000000.0, 16)), "mlp": dense(160)},
            {"type": "attention", "mixer": attn(4, 1, 64, 64, 0.1, (50000.0, 64), 70), "mlp": dense(96)},
            {"type": "gla", "mixer": gla(2, 64, 64, 16.0, 16), "mlp": dense(64)},
            {"type": "attention", "mixer": attn(2, 1, 64, 48, 0.12, (777.0, 32), 129, 5), "mlp": None},
        ]}),
    "riv-c": dict(seed=43, block_size=8, cfg={
        "architecture": "Rivetar", "vocab": 97, "width": 40, "norm": {"eps": 1e-4}, "embedding": {"scale": 4.0},
        "logit_softcap": 7.5, "loop": {"start": 0, "stop": 3, "times": 2},
        "layers": [
            {"type": "gla", "mixer": gla(1, 10, 14, 1.0, 3), "mlp": dense(24)},
            {"type": "attention", "mixer": attn(3, 1, 20, 12, 0.35, (50.0, 6), 9, 12), "mlp": None},
            {"type": "latent_attention", "mixer": latent(5, 6, 6, 10, 12, 10, 0.45, (20.0, 2)), "mlp": None},
        ]}),
}

TORCH_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def write_model_from(cfg_dict: dict, seed: int, dtype: str, folder: str, head_scale: float = 40.0) -> str:
    """Random weights through the package's own writer; the output head is scaled up so that the logits
    spread over several units and the cap on them (where the model has one) bends them."""
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
