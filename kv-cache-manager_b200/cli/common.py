"""What the command-line tools share: building an engine from the reference's flag names."""
from __future__ import annotations

import os
import tempfile


def engine_config_from_args(a):
    """Flags as the reference's kvbench (``src/main_bench.cpp:24-42``) plus this engine's own."""
    from ..config import EngineConfig, KVManagerConfig, SchedulerConfig, canonical_dtype
    kv = KVManagerConfig(policy=a.str("policy", "paged"), block_size=a.i32("block-size", 16),
                         max_seq_len=a.i32("max-seq-len", 2048), prefix_caching=a.flag("prefix"),
                         num_blocks=a.i32("num-blocks", 0), watermark_blocks=a.i32("watermark", -1))
    sc = SchedulerConfig(max_num_seqs=a.i32("max-num-seqs", 256),
                         max_batched_tokens=a.i32("max-batched-tokens", 4096),
                         prefill_chunk=a.i32("prefill-chunk", 0),
                         chunked_prefill=not a.flag("no-chunked-prefill"))
    return EngineConfig(kv=kv, pool_gb=a.f64("pool-gb", 1.0), sched=sc,
                        dtype=canonical_dtype(a.str("dtype", "bfloat16")), attn=a.str("attn", "auto"), gemm=a.str("gemm", "auto"),
                        sampling_seed=a.i64("sampling-seed", 0), cuda_graphs=not a.flag("no-graphs"))


def _tolanex_mini():
    """A small Tolanex: delta, latent attention, a latent layer reading the one before, delta; experts on
    three of the four layers."""
    def mlp(shared):
        m = {"kind": "moe", "expert": {"ff": 128},
             "router": {"experts": 16, "top": 2, "scale": 1.5, "groups": {"count": 4, "keep": 2}}}
        if shared:
            m["shared"] = {"ff": shared}
        return m
    return {"architecture": "Tolanex", "vocab": 1000, "width": 384, "max_positions": 1024, "norm": {"eps": 1e-5},
            "residual_mult": 0.6, "embedding": {"bigram": {"buckets": 1021, "mul_prev": 31, "mul_cur": 7}},
            "layers": [
                {"type": "delta", "mixer": {"heads": 6, "kv_heads": 3, "dim": 64, "vdim": 64, "conv": 4}, "mlp": mlp(256)},
                {"type": "latent_attention", "mixer": {"heads": 6, "dim": 32, "vdim": 64, "kv_rank": 64, "scale": 0.18},
                 "mlp": mlp(0)},
                {"type": "latent_attention", "mixer": {"heads": 4, "dim": 32, "vdim": 32, "kv_rank": 64, "scale": 0.18,
                                                        "kv_from": 1}, "mlp": None},
                {"type": "delta", "mixer": {"heads": 4, "kv_heads": 4, "dim": 32, "vdim": 96, "conv": 2}, "mlp": mlp(128)},
            ]}


def _bifatar_mini():
    """A small Bifatar: windowed attention (values kept), the state-space mixer, attention beside the
    channel-decay delta rule, windowed attention that mixes the first layer's values."""
    def attn(window, base):
        return {"heads": 6, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.1, "rot": {"base": base, "dims": 32},
                "mask": {"size": window}, "softcap": 25.0, "v_mix": True}
    dense = {"kind": "dense", "ff": 768}
    return {"architecture": "Bifatar", "vocab": 1000, "width": 384, "norm": {"eps": 1e-5},
            "layers": [
                {"type": "attention", "mixer": attn(200, 10000.0), "mlp": dense},
                {"type": "mamba2", "mixer": {"heads": 12, "vdim": 64, "state": 64, "groups": 2, "conv": 4, "norm_groups": 2},
                 "mlp": dense},
                {"type": "parallel", "mixer": {
                    "left": {"heads": 6, "kv_heads": 2, "dim": 64, "vdim": 32, "scale": 0.125, "rot": {"base": 500000.0, "dims": 64}},
                    "right": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 96, "conv": 3, "decay_rank": 16, "gate_rank": 24},
                    "left_scale": 1.0, "right_scale": 0.5}, "mlp": None},
                {"type": "attention", "mixer": attn(72, 50000.0), "mlp": dense},
            ]}


def _rivetar_mini():
    """A small Rivetar: attention over a cached latent with a rotated key part, a looped span of gated linear
    attention and windowed attention that keeps the first tokens, a latent layer behind the loop."""
    dense = {"kind": "dense", "ff": 640}
    latent = {"heads": 6, "dim": 48, "rot_dim": 32, "vdim": 64, "kv_rank": 96, "q_rank": 160, "scale": 0.11,
              "rot": {"base": 100000.0, "dims": 32}}
    return {"architecture": "Rivetar", "vocab": 1000, "width": 384, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
            "logit_softcap": 25.0, "loop": {"start": 1, "stop": 3, "times": 2},
            "layers": [
                {"type": "latent_attention", "mixer": latent, "mlp": dense},
                {"type": "gla", "mixer": {"heads": 6, "dim": 32, "vdim": 64, "tau": 8.0, "decay_rank": 24}, "mlp": None},
                {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 64, "vdim": 32, "scale": 0.125,
                                                "rot": {"base": 10000.0, "dims": 32}, "mask": {"size": 90, "keep_first": 3}},
                 "mlp": dense},
                {"type": "latent_attention", "mixer": latent, "mlp": dense},
            ]}


def _lobutar_mini():
    """A small Lobutar: three residual streams; differential attention with a dense feed-forward, run a second time
    with the same weights behind a windowed latent layer with grouped experts; a latent layer without a window."""
    attn = {"heads": 6, "kv_heads": 2, "dim": 32, "vdim": 64, "diff": 0.4, "scale": 0.18, "rot": {"base": 10000.0, "dims": 16}}
    latent = {"heads": 6, "dim": 48, "rot_dim": 32, "vdim": 64, "kv_rank": 96, "scale": 0.11, "rot": {"base": 100000.0, "dims": 32}}
    moe = {"kind": "moe", "expert": {"ff": 128}, "shared": {"ff": 256},
           "router": {"experts": 16, "top": 3, "scale": 1.5, "groups": {"count": 4, "keep": 2}}}
    first = {"type": "attention", "mixer": attn, "mlp": {"kind": "dense", "ff": 640}}
    return {"architecture": "Lobutar", "vocab": 1000, "width": 384, "norm": {"eps": 1e-5}, "streams": 3,
            "layers": [
                first,
                {"type": "latent_attention", "mixer": dict(latent, mask={"size": 90}), "mlp": moe},
                dict(first, weights_of=0),
                {"type": "latent_attention", "mixer": latent, "mlp": None},
            ]}


PRESETS = {
    # name: (config.json keys, seed, norm jitter); keys with "architecture" go through the registry,
    # the others are those of a Llama dense decoder
    "tolanex-mini": (_tolanex_mini(), 4, 0.1),
    "bifatar-mini": (_bifatar_mini(), 5, 0.1),
    "rivetar-mini": (_rivetar_mini(), 7, 0.1),
    "lobutar-mini": (_lobutar_mini(), 8, 0.1),
    "tiny-a": (dict(vocab_size=256, hidden_size=64, intermediate_size=172, num_hidden_layers=2,
                    num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=128,
                    rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False), 0, 0.0),
    "tiny-b": (dict(vocab_size=384, hidden_size=96, intermediate_size=256, num_hidden_layers=3,
                    num_attention_heads=3, num_key_value_heads=1, head_dim=32, max_position_embeddings=256,
                    rope_theta=500000.0, rms_norm_eps=1e-6, tie_word_embeddings=True), 1, 0.1),
    "tiny-c": (dict(vocab_size=320, hidden_size=136, intermediate_size=344, num_hidden_layers=2,
                    num_attention_heads=3, num_key_value_heads=1, head_dim=64, max_position_embeddings=512,
                    rope_theta=250000.0, rms_norm_eps=2e-6, tie_word_embeddings=False), 2, 0.05),
    "tinyllama-1.1b": (dict(vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22,
                            num_attention_heads=32, num_key_value_heads=4, head_dim=64,
                            max_position_embeddings=2048, rope_theta=10000.0, rms_norm_eps=1e-5,
                            tie_word_embeddings=False), 0, 0.0),
    "llama-2-7b": (dict(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                        num_attention_heads=32, num_key_value_heads=32, head_dim=128,
                        max_position_embeddings=4096, rope_theta=10000.0, rms_norm_eps=1e-5,
                        tie_word_embeddings=False), 0, 0.0),
    "llama-3-8b": (dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                        num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                        max_position_embeddings=8192, rope_theta=500000.0, rms_norm_eps=1e-5,
                        tie_word_embeddings=False), 0, 0.0),
}


def load_model_from_args(a, dtype: str, device: str = "cuda:0", stored_as: str = ""):
    """``--model DIR`` (config.json + model.safetensors) or ``--preset NAME [--random-seed S]``
    (random weights of a named shape, generated on the device).  ``stored_as``: the random weights
    are rounded to that type first, as if read from a checkpoint stored in it (a float32 model with
    the very values of the bfloat16 one)."""
    import torch
    from ..config import LlamaConfig
    from ..engine import load_model, model_from_tensors, torch_dtype
    from ..weights import random_tensors
    folder = a.str("model", "")
    preset = a.str("preset", "")
    if folder:
        return load_model(folder, dtype, device)
    if not preset:
        raise SystemExit("give --model DIR or --preset NAME (" + ", ".join(PRESETS) + ")")
    if preset not in PRESETS:
        raise SystemExit(f"unknown preset '{preset}'; known: {', '.join(PRESETS)}")
    keys, seed, jitter = PRESETS[preset]
    if "architecture" in keys:
        from ..config import config_from_dict
        cfg = config_from_dict(keys)
    else:
        cfg = LlamaConfig(architecture="LlamaForCausalLM", **keys)
    seed = a.i64("random-seed", seed)
    tensors = dict(random_tensors(cfg, seed, torch_dtype(stored_as or dtype), device=device, norm_jitter=jitter))
    if stored_as and stored_as != dtype:
        tensors = {k: v.to(torch_dtype(dtype)) for k, v in tensors.items()}
    return model_from_tensors(cfg, tensors, dtype, device)
