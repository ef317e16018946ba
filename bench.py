#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second at TinyLlama-1.1B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A *step* is one decode step of the whole batch.  The default run has the layer sizes of the
reference's benchmark model (TinyLlama 1.1B: 22 layers, hidden 2048, 32 query / 4 KV heads of
64, FFN 5632, vocabulary 32000) with random bfloat16 weights, a batch of 8 requests with
1,024-token prompts that are decoded towards 2,048 tokens.  It prints ONE JSON line:

* ``value``     decoded tokens per second, from CUDA events around the device work of each of
                the K timed steps (kernels of the step, without the host's batch building);
* ``e2e``       the same K steps through the Python entry point (``Engine.step``): host tokens in
                through one pinned host-to-device copy per step, sampled tokens read back;
* ``prefill``   one 2,048-token prompt in one step: tokens/s, ms and fraction of the bf16 peak;
* ``roofline``  bytes the decode step must read (every weight once, the cache of the live
                requests) over its time, against the HBM copy bandwidth;
* ``points``    decode tokens/s at batch 1 and 64, each with the same roofline fraction
                (``decode_b1_hbm_frac``, ``decode_b64_hbm_frac``).

The timed decode window is centred on a context of 1,536 tokens (the middle of 1,024 -> 2,048)
whatever K is: prompts have ``1536 - W - K/2`` tokens, which is 1,020 for the default K = 1,000.

This engine is single-GPU: for ``--gpus N`` with N > 1 it says so and exits with 2.  The
reference arm (``--impl reference``) runs the unmodified reference, built by its own CMake project
under ``baseline/_ref``, through its serving benchmark ``kvbench`` on a random weight file of the
same shape, with the same prompts lengths, batch and steps (``baseline/reference_arm.py``); it
prints the same JSON line with ``"impl": "reference"``, or one ``unavailable`` line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Layer sizes of the benchmark model (the reference's TinyLlama-1.1B, docs/design.md:3-7).
MODEL = dict(vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22,
             num_attention_heads=32, num_key_value_heads=4, head_dim=64,
             max_position_embeddings=2048, rope_theta=10000.0, rms_norm_eps=1e-5,
             tie_word_embeddings=False)
PROMPT_LEN = 1024          # of the metric; the run's own prompt length centres the timed window
MID_CONTEXT = 1536         # middle of 1,024 -> 2,048
CONTEXT = 2048
PREFILL_TOKENS = 2048
BLOCK_SIZE = 16
# Reference numbers (RTX 4080, its own trace): decode tokens/s at batch 1 / 8 / 64.
PUBLISHED = {1: 222.0, 8: 1643.0, 64: 9257.0}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS, source="fallback")
    try:
        with open(p) as f:
            d = json.load(f)
        for k in FALLBACK_PEAKS:
            if isinstance(d.get(k), (int, float)) and d[k] > 0:
                out[k] = float(d[k])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = [int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6
                          for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": int(statistics.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm)}


def model_bytes_and_flops(cfg, layers):
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = (cfg.qkv_dim * H + H * cfg.q_dim + 2 * I * H + H * I)
    weights = per_layer * layers + V * H                       # matrices read by a decode step
    norms = (2 * layers + 1) * H
    kv_per_token = 2 * layers * cfg.kv_dim
    return dict(matrix_params=weights, weight_bytes=2 * (weights + norms),
                kv_bytes_per_token=2 * kv_per_token, per_layer_params=per_layer)


def build_engine(layers, batch, max_len, graphs=True, max_batched=4096):
    import torch
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, LlamaConfig, SchedulerConfig
    from kvcm.engine import Engine, model_from_tensors
    from kvcm.weights import random_tensors
    cfg = LlamaConfig(architecture="LlamaForCausalLM", **dict(MODEL, num_hidden_layers=layers))
    tensors = dict(random_tensors(cfg, 0, torch.bfloat16, device="cuda:0"))
    spec = model_from_tensors(cfg, tensors, "bfloat16", "cuda:0")
    del tensors
    pages = batch * ((max_len + BLOCK_SIZE - 1) // BLOCK_SIZE + 1) + 8
    ec = EngineConfig(kv=KVManagerConfig(num_blocks=pages, block_size=BLOCK_SIZE, max_seq_len=max_len,
                                         watermark_blocks=0),
                      sched=SchedulerConfig(max_num_seqs=max(batch, 8), max_batched_tokens=max_batched),
                      dtype="bfloat16", cuda_graphs=graphs)
    return cfg, spec, ec


def window_prompt_len(steps, warmup):
    """Prompt length that puts the middle of the timed steps at a context of MID_CONTEXT tokens."""
    return max(16, MID_CONTEXT - warmup - steps // 2)


def decode_run(spec, ec, vocab, batch, steps, warmup, prompt_len, sample_clocks=False):
    """Prefills `batch` prompts of `prompt_len` tokens, runs `warmup` untimed and `steps` timed decode
    steps through Engine.step().  Returns device ms, wall ms, copies per step, launches per step."""
    import torch
    from kvcm.engine.engine import DeviceTimer, Engine
    from kvcm.kernels import launch_count
    eng = Engine(spec, ec)
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(3, vocab, (batch, prompt_len), generator=g).tolist()
    for p in prompts:
        eng.add_request(p, max_new_tokens=1 << 30)   # ends only at max_seq_len, sized with headroom
    while eng.sched.num_waiting() or eng.sched.counters().prefill_tokens < batch * prompt_len:
        eng.step()                                   # prompt portions (and the first tokens)
    for _ in range(warmup):
        info = eng.step()
    assert info.decode_seqs == batch and info.prefill_tokens == 0, "warm-up must end in pure decoding"
    torch.cuda.synchronize()
    clocks = ClockSampler()
    if sample_clocks:
        clocks.start()
        time.sleep(0.25)
    timer = DeviceTimer()
    eng.device_timer = timer
    h2d = d2h = 0
    launches0 = launch_count()
    graph_kernels = 0
    ctx_sum = 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        info = eng.step()
        h2d += info.h2d_bytes
        d2h += info.d2h_bytes
        if info.graph and eng.native is None:
            graph_kernels += eng.graphs.kernels_last       # (the C++ loop reports its launches itself)
        ctx_sum += eng.sched.cached_tokens_total()
    wall_ms = (time.perf_counter() - t0) * 1e3     # the host holds the tokens of `steps` steps
    dev_ms = timer.total_ms()                      # device time of exactly these steps
    if eng.native is not None:
        eng.native.drain()                         # (a step enqueued ahead ends outside the timed region)
    torch.cuda.synchronize()
    eager_kernels = launch_count() - launches0
    eng.device_timer = None
    clk = clocks.stop() if sample_clocks else None
    assert info.decode_seqs == batch, f"a request ended inside the timed region: {info}"
    res = dict(dev_ms=dev_ms, wall_ms=wall_ms, h2d=h2d / steps, d2h=d2h / steps,
               launches=graph_kernels + eager_kernels, mean_ctx=ctx_sum / (steps * batch), clocks=clk,
               graph_steps=eng.graphs.replays if eng.graphs else 0)
    del eng
    torch.cuda.empty_cache()
    return res


def prefill_run(spec, ec, vocab, cfg, layers, reps=5):
    """One prompt of PREFILL_TOKENS tokens in one step.  Returns (device ms, flops, end-to-end ms): the
    device time of the step's kernels from CUDA events, and the wall time of the same step through
    ``Engine.add_request`` + ``Engine.step`` (host tokens in, the first sampled token out)."""
    import torch
    from kvcm.engine.engine import DeviceTimer, Engine
    eng = Engine(spec, ec)
    g = torch.Generator().manual_seed(2)
    dev, wall = [], []
    for r in range(reps + 2):
        toks = torch.randint(3, vocab, (PREFILL_TOKENS,), generator=g).tolist()
        timer = DeviceTimer()
        eng.device_timer = timer
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.add_request(toks, max_new_tokens=1)
        info = eng.step()
        t1 = time.perf_counter()
        assert info.prefill_tokens == PREFILL_TOKENS and info.sampled == 1, info
        eng.take_finished()
        ms = timer.total_ms()
        eng.device_timer = None
        if r >= 2:
            dev.append(ms)
            wall.append((t1 - t0) * 1e3)
    m = model_bytes_and_flops(cfg, layers)
    T = PREFILL_TOKENS
    gemm_flops = 2.0 * m["per_layer_params"] * layers * T + 2.0 * cfg.vocab_size * cfg.hidden_size
    attn_flops = 4.0 * cfg.head_dim * cfg.num_attention_heads * (T * (T + 1) / 2) * layers
    del eng
    torch.cuda.empty_cache()
    return statistics.median(dev), gemm_flops + attn_flops, statistics.median(wall)

# ------------------------------------------------------------------------------------------------
# --compare tolanex: the Tolanex design beside the Llama decoder at equal width, depth and active
# feed-forward size (random bfloat16 weights): prefill of one 2,048-token prompt and decode steps
# of 8 requests at a context of about 1,024, device time from CUDA events, and the device time of
# every kernel family of one eager step of each kind with what that family has to compute or move.

COMPARE_SIZES = {
    # width, layers, heads x head size, latent rank, experts / top / expert ff / groups, shared ff
    "w2048": dict(width=2048, layers=4, heads=16, dim=128, rank=128, experts=32, top=4, ff=512, groups=(4, 2), shared=1024,
                  kv_heads=4),
    "w4096": dict(width=4096, layers=2, heads=32, dim=128, rank=256, experts=64, top=6, ff=1024, groups=(8, 4), shared=2048,
                  kv_heads=8),
}
COMPARE_VOCAB = 32000


def compare_configs(z):
    """(Tolanex config, Llama config) of one size.  Tolanex layers alternate delta / latent attention;
    every second latent layer reads the pages of the one before it."""
    from kvcm.config import LlamaConfig, config_from_dict
    D, H, d = z["width"], z["heads"], z["dim"]
    mlp = {"kind": "moe", "expert": {"ff": z["ff"]}, "shared": {"ff": z["shared"]},
           "router": {"experts": z["experts"], "top": z["top"], "scale": 1.0,
                      "groups": {"count": z["groups"][0], "keep": z["groups"][1]}}}
    layers, last_latent, latents = [], None, 0
    for i in range(z["layers"]):
        if i % 2 == 0:
            layers.append({"type": "delta", "mixer": {"heads": H, "kv_heads": H // 2, "dim": d, "vdim": d, "conv": 4}, "mlp": mlp})
        else:
            m = {"heads": H, "dim": d, "vdim": d, "kv_rank": z["rank"], "scale": d ** -0.5}
            if latents % 2 == 1:
                m["kv_from"] = last_latent
            else:
                last_latent = i
            latents += 1
            layers.append({"type": "latent_attention", "mixer": m, "mlp": mlp})
    tol = config_from_dict({"architecture": "Tolanex", "vocab": COMPARE_VOCAB, "width": D, "max_positions": 4096,
                            "norm": {"eps": 1e-6}, "residual_mult": 0.5,
                            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 127, "mul_cur": 17}}, "layers": layers})
    active_ff = z["top"] * z["ff"] + z["shared"]
    lla = LlamaConfig(architecture="LlamaForCausalLM", vocab_size=COMPARE_VOCAB, hidden_size=D, intermediate_size=active_ff,
                      num_hidden_layers=z["layers"], num_attention_heads=H, num_key_value_heads=z["kv_heads"], head_dim=d,
                      max_position_embeddings=4096, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)
    return tol, lla


def family_profile(spec, vocab, kind):
    """Device ms per kernel family of ONE eager step: kind 'prefill' (one prompt of 2,048 tokens) or
    'decode' (8 requests with 1,024 cached tokens, one token each)."""
    import torch
    from kvcm.engine.replay import ReplaySession
    from kvcm.kernels import library as K
    s = ReplaySession(spec, "bfloat16", 8 * 1088 + 2112, block_size=BLOCK_SIZE, max_live=9)
    g = torch.Generator().manual_seed(5)
    if kind == "prefill":
        toks = torch.randint(3, vocab, (3, PREFILL_TOKENS), generator=g).tolist()
        for i in range(2):
            s.step([dict(id=f"w{i}", tokens=toks[i], want=[PREFILL_TOKENS - 1])], end=[f"w{i}"])
        torch.cuda.synchronize()
        K.profile_start()
        s.step([dict(id="p", tokens=toks[2], want=[PREFILL_TOKENS - 1])], end=["p"])
        return K.profile_stop()
    toks = torch.randint(3, vocab, (8, 1024 + 3), generator=g).tolist()
    for i in range(8):
        s.step([dict(id=i, tokens=toks[i][:1024], want=[])])
    for k in range(2):
        s.step([dict(id=i, tokens=[toks[i][1024 + k]], want=[0]) for i in range(8)])
    torch.cuda.synchronize()
    K.profile_start()
    s.step([dict(id=i, tokens=[toks[i][1026]], want=[0]) for i in range(8)])
    return K.profile_stop()


def tolanex_work(z, T, ctx, decode):
    """What the families of one Tolanex step have to do at least: flops, or bytes they must move."""
    D, H, d, R, E, top, F = z["width"], z["heads"], z["dim"], z["rank"], z["experts"], z["top"], z["ff"]
    n_delta, n_latent = (z["layers"] + 1) // 2, z["layers"] // 2
    hit = min(E, T * top)                                        # experts that get a row, at most
    return {
        "moe_experts_tcgen05": dict(flops=2.0 * T * top * 3 * F * D * z["layers"],
                                    bytes=2.0 * hit * 3 * F * D * z["layers"] if decode else None),
        "delta_scan": dict(flops=6.0 * T * H * d * d * n_delta,                      # two dot products and one update a token
                           bytes=(8.0 if decode else 0.0) * T * H * d * d * n_delta if decode else None),   # state read + written
        "attention": dict(flops=4.0 * R * H * (T * ctx if decode else T * (T + 1) / 2) * n_latent,
                          bytes=2.0 * T * ctx * R * n_latent if decode else None),
    }


def llama_work(z, T, ctx, decode):
    D, H, d = z["width"], z["heads"], z["dim"]
    I = z["top"] * z["ff"] + z["shared"]
    L = z["layers"]
    return {
        "feed_forward": dict(flops=2.0 * T * 3 * I * D * L, bytes=2.0 * 3 * I * D * L if decode else None),
        "attention": dict(flops=4.0 * d * H * (T * ctx if decode else T * (T + 1) / 2) * L,
                          bytes=2.0 * 2 * T * ctx * z["kv_heads"] * d * L if decode else None),
    }



# --compare bifatar: the Bifatar design (windowed attention with sink, cap and value mixing; the state-space
# mixer; attention beside the channel-decay delta rule; tanh norms, one per layer; squared-ReLU feed-forward)
# beside the Llama decoder at equal width, depth, head count and feed-forward parameter count.
BIFATAR_SIZES = {
    "b2048": dict(width=2048, order=("attention", "mamba2", "parallel", "attention"), heads=16, kv_heads=4, dim=128, window=1024,
                  ssm_heads=64, ssm_vdim=64, ssm_state=128, ssm_groups=8, delta_heads=16, llama_ff=4096),
    "b4096": dict(width=4096, order=("attention", "mamba2", "parallel"), heads=32, kv_heads=8, dim=128, window=1024,
                  ssm_heads=128, ssm_vdim=64, ssm_state=128, ssm_groups=8, delta_heads=32, llama_ff=8192),
}


def bifatar_configs(z):
    """(Bifatar config, Llama config) of one size.  The ungated feed-forward has two matrices where the gated
    one has three: its inner size is 1.5 times Llama's, so that both read and multiply the same weights."""
    from kvcm.config import LlamaConfig, config_from_dict
    D, H, G, d = z["width"], z["heads"], z["kv_heads"], z["dim"]
    mlp = {"kind": "dense", "ff": z["llama_ff"] * 3 // 2}
    rot = {"base": 10000.0, "dims": d}
    layers = []
    for kind in z["order"]:
        if kind == "attention":
            m = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5 / 4, "rot": rot, "mask": {"size": z["window"]},
                 "softcap": 30.0, "v_mix": True}
        elif kind == "mamba2":
            m = {"heads": z["ssm_heads"], "vdim": z["ssm_vdim"], "state": z["ssm_state"], "groups": z["ssm_groups"], "conv": 4,
                 "norm_groups": z["ssm_groups"]}
        else:
            m = {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5, "rot": rot},
                 "right": {"heads": z["delta_heads"], "kv_heads": z["delta_heads"], "dim": d, "vdim": d, "conv": 4,
                           "decay_rank": 64, "gate_rank": 64},
                 "left_scale": 1.0, "right_scale": 1.0}
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    bif = config_from_dict({"architecture": "Bifatar", "vocab": COMPARE_VOCAB, "width": D, "norm": {"eps": 1e-6}, "layers": layers})
    lla = LlamaConfig(architecture="LlamaForCausalLM", vocab_size=COMPARE_VOCAB, hidden_size=D, intermediate_size=z["llama_ff"],
                      num_hidden_layers=len(layers), num_attention_heads=H, num_key_value_heads=G, head_dim=d,
                      max_position_embeddings=4096, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)
    return bif, lla


def bifatar_work(z, T, ctx, decode):
    """What the families of one Bifatar step have to do at least: flops, or bytes they must move."""
    D, H, G, d, W = z["width"], z["heads"], z["kv_heads"], z["dim"], z["window"]
    n_win = sum(k == "attention" for k in z["order"])
    n_par = sum(k == "parallel" for k in z["order"])
    n_ssm = sum(k == "mamba2" for k in z["order"])
    L = len(z["order"])
    seen_win = T * min(ctx, W) if decode else sum(min(i + 1, W) for i in range(T))
    seen_all = T * ctx if decode else T * (T + 1) / 2
    ssm_state = z["ssm_heads"] * z["ssm_state"] * z["ssm_vdim"]
    delta_state = z["delta_heads"] * d * d
    ff = z["llama_ff"] * 3 // 2
    return {
        "attention": dict(flops=4.0 * d * H * (seen_win * n_win + seen_all * n_par),
                          bytes=2.0 * 2 * G * d * (T * min(ctx, W) * n_win + T * ctx * n_par) if decode else None),
        "state_scan": dict(flops=T * (4.0 * ssm_state * n_ssm + 7.0 * delta_state * n_par),
                           bytes=8.0 * T * (ssm_state * n_ssm + delta_state * n_par) if decode else None),
        "feed_forward": dict(flops=2.0 * T * 2 * ff * D * L, bytes=2.0 * 2 * ff * D * L if decode else None),
        "dyt_norm": dict(flops=None, bytes=T * D * (4.0 * 2 + 4.0 * 2.3 + 2.0) * L),
    }


# --compare rivetar: the Rivetar design (attention over a cached latent with a rotated key part; gated linear
# attention; windowed attention with kept first tokens, a sink and turned values; norms on both sides of every
# sublayer; PolyNorm feed-forward; a looped span of layers) beside the Llama decoder at equal width, number of
# layer runs, head count and feed-forward parameter count.
RIVETAR_SIZES = {
    "r2048": dict(width=2048, order=("latent_attention", "gla", "attention", "latent_attention"), loop=None, heads=16, kv_heads=4,
                  dim=128, rot_dim=64, kv_rank=192, q_rank=768, window=1024, keep_first=4, gla_heads=16, llama_ff=4096),
    "r4096": dict(width=4096, order=("latent_attention", "gla", "attention"), loop=(0, 2, 2), heads=32, kv_heads=8, dim=128,
                  rot_dim=64, kv_rank=192, q_rank=1536, window=1024, keep_first=4, gla_heads=32, llama_ff=8192),
}


def rivetar_runs(z):
    """The layer kinds in the order in which they run (a looped span counts every pass)."""
    order = list(z["order"])
    if z["loop"]:
        a, b, times = z["loop"]
        order = order[:a] + order[a:b] * times + order[b:]
    return order


def rivetar_configs(z):
    """(Rivetar config, Llama config) of one size.  The ungated feed-forward has two matrices where the gated one
    has three: its inner size is 1.5 times Llama's.  Llama gets as many layers as Rivetar has layer runs."""
    from kvcm.config import LlamaConfig, config_from_dict
    D, H, G, d = z["width"], z["heads"], z["kv_heads"], z["dim"]
    mlp = {"kind": "dense", "ff": z["llama_ff"] * 3 // 2}
    layers = []
    for kind in z["order"]:
        if kind == "attention":
            m = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5, "rot": {"base": 10000.0, "dims": d // 2},
                 "mask": {"size": z["window"], "keep_first": z["keep_first"]}}
        elif kind == "gla":
            m = {"heads": z["gla_heads"], "dim": d, "vdim": d, "tau": 16.0, "decay_rank": 64}
        else:
            m = {"heads": H, "dim": d, "rot_dim": z["rot_dim"], "vdim": d, "kv_rank": z["kv_rank"], "q_rank": z["q_rank"],
                 "scale": (d + z["rot_dim"]) ** -0.5, "rot": {"base": 10000.0, "dims": z["rot_dim"]}}
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    top = {"architecture": "Rivetar", "vocab": COMPARE_VOCAB, "width": D, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
           "logit_softcap": 30.0, "layers": layers}
    if z["loop"]:
        top["loop"] = dict(zip(("start", "stop", "times"), z["loop"]))
    riv = config_from_dict(top)
    lla = LlamaConfig(architecture="LlamaForCausalLM", vocab_size=COMPARE_VOCAB, hidden_size=D, intermediate_size=z["llama_ff"],
                      num_hidden_layers=len(rivetar_runs(z)), num_attention_heads=H, num_key_value_heads=G, head_dim=d,
                      max_position_embeddings=4096, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)
    return riv, lla


def rivetar_work(z, T, ctx, decode):
    """What the families of one Rivetar step have to do at least: flops, or bytes they must move."""
    D, H, G, d, W = z["width"], z["heads"], z["kv_heads"], z["dim"], z["window"]
    runs = rivetar_runs(z)
    n_win, n_lat, n_gla, L = runs.count("attention"), runs.count("latent_attention"), runs.count("gla"), len(runs)
    seen_win = T * min(ctx, W + z["keep_first"]) if decode else sum(min(i + 1, W + z["keep_first"]) for i in range(T))
    seen_all = T * ctx if decode else T * (T + 1) / 2
    lat = z["kv_rank"] + z["rot_dim"]
    state = z["gla_heads"] * d * d
    ff = z["llama_ff"] * 3 // 2
    return {
        "attention": dict(flops=4.0 * H * (d * seen_win * n_win + lat * seen_all * n_lat),
                          bytes=2.0 * (2 * G * d * T * min(ctx, W) * n_win + lat * T * ctx * n_lat) if decode else None),
        "state_scan": dict(flops=T * 4.0 * state * n_gla, bytes=8.0 * T * state * n_gla if decode else None),
        "feed_forward": dict(flops=2.0 * T * 2 * ff * D * L, bytes=2.0 * 2 * ff * D * L if decode else None),
        "norm_post_pre": dict(flops=None, bytes=T * D * (4.0 * 3 + 2.0) * 2 * L),
        "poly_norm_act": dict(flops=None, bytes=T * ff * (4.0 + 2.0) * L),
    }


# --compare lobutar: the Lobutar design (several residual streams; differential attention; windowed attention over a
# cached latent with a sink and an output gate; dense feed-forward or routed experts with a shared one; a layer run a
# second time with the same weights) beside the Llama decoder at equal width, number of layer runs, head count and
# active feed-forward size.
LOBUTAR_SIZES = {
    "h2048": dict(width=2048, streams=4, order=("attention", "latent_attention", "attention", "latent_attention"), shared_run=(2, 0),
                  heads=16, kv_heads=4, dim=128, map_dim=64, rot_dim=64, kv_rank=192, window=1024, experts=32, moe_top=6,
                  expert_ff=512, groups=(4, 2), moe_shared=1024, llama_ff=4096),
    "h4096": dict(width=4096, streams=4, order=("attention", "latent_attention", "latent_attention"), shared_run=(2, 1),
                  heads=32, kv_heads=8, dim=128, map_dim=64, rot_dim=64, kv_rank=192, window=1024, experts=64, moe_top=6,
                  expert_ff=1024, groups=(8, 4), moe_shared=2048, llama_ff=8192),
}


def lobutar_configs(z):
    """(Lobutar config, Llama config) of one size.  Attention layers carry the dense feed-forward, latent layers the
    experts (chosen plus shared = Llama's inner size); ``shared_run`` = (i, j): layer i runs with layer j's weights.
    A differential head has two maps of ``map_dim`` and values of ``dim``: its cached key pair is as long as a
    Llama key.  Llama gets as many layers as Lobutar has layer runs."""
    from kvcm.config import LlamaConfig, config_from_dict
    D, H, G, d = z["width"], z["heads"], z["kv_heads"], z["dim"]
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "shared": {"ff": z["moe_shared"]},
           "router": {"experts": z["experts"], "top": z["moe_top"], "scale": 2.0,
                      "groups": {"count": z["groups"][0], "keep": z["groups"][1]}}}
    layers = []
    for kind in z["order"]:
        if kind == "attention":
            m = {"heads": H, "kv_heads": G, "dim": z["map_dim"], "vdim": d, "diff": 0.5, "scale": z["map_dim"] ** -0.5,
                 "rot": {"base": 10000.0, "dims": z["map_dim"] // 2}}
            layers.append({"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": z["llama_ff"]}})
        else:
            m = {"heads": H, "dim": d, "rot_dim": z["rot_dim"], "vdim": d, "kv_rank": z["kv_rank"], "scale": (d + z["rot_dim"]) ** -0.5,
                 "rot": {"base": 10000.0, "dims": z["rot_dim"]}, "mask": {"size": z["window"]}}
            layers.append({"type": kind, "mixer": m, "mlp": moe})
    i, j = z["shared_run"]
    layers[i] = dict(layers[j], weights_of=j)
    lob = config_from_dict({"architecture": "Lobutar", "vocab": COMPARE_VOCAB, "width": D, "norm": {"eps": 1e-6},
                            "streams": z["streams"], "layers": layers})
    lla = LlamaConfig(architecture="LlamaForCausalLM", vocab_size=COMPARE_VOCAB, hidden_size=D, intermediate_size=z["llama_ff"],
                      num_hidden_layers=len(z["order"]), num_attention_heads=H, num_key_value_heads=G, head_dim=d,
                      max_position_embeddings=4096, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)
    return lob, lla


def lobutar_work(z, T, ctx, decode):
    """What the families of one Lobutar step have to do at least: flops, or bytes they must move."""
    D, H, G, d, W, S = z["width"], z["heads"], z["kv_heads"], z["dim"], z["window"], z["streams"]
    runs = list(z["order"])
    n_att, n_lat, L = runs.count("attention"), runs.count("latent_attention"), len(runs)
    seen_all = T * ctx if decode else T * (T + 1) / 2
    seen_win = T * min(ctx, W) if decode else sum(min(i + 1, W) for i in range(T))
    lat = z["kv_rank"] + z["rot_dim"]
    hit = min(z["experts"], T * z["moe_top"])
    return {
        # two maps a head: two score products over map_dim and two weighted sums over the values
        "attention": dict(flops=4.0 * H * ((z["map_dim"] + d) * 2 * seen_all * n_att + lat * seen_win * n_lat),
                          bytes=2.0 * ((2 * z["map_dim"] + d) * G * T * ctx * n_att + lat * T * min(ctx, W) * n_lat) if decode else None),
        "moe_experts_tcgen05": dict(flops=2.0 * T * z["moe_top"] * 3 * z["expert_ff"] * D * n_lat,
                                    bytes=2.0 * hit * 3 * z["expert_ff"] * D * n_lat if decode else None),
        "feed_forward": dict(flops=2.0 * T * 3 * (z["llama_ff"] * n_att + z["moe_shared"] * n_lat) * D,
                             bytes=2.0 * 3 * (z["llama_ff"] * n_att + z["moe_shared"] * n_lat) * D if decode else None),
        # the streams are read and written once per sublayer, the sublayer's output read, its input written
        "hc_step": dict(flops=None, bytes=T * D * (4.0 * 2 * S + 4.0 + 2.0) * 2 * L),
        "diff_combine": dict(flops=None, bytes=T * H * d * 2.0 * 3 * n_att),
    }


def compare_main(args) -> int:
    import torch
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    from kvcm.engine import model_from_tensors
    from kvcm.weights import random_tensors
    pk = peaks()
    first = args.compare
    sizes, configs, first_work = {"bifatar": (BIFATAR_SIZES, bifatar_configs, bifatar_work),
                                  "rivetar": (RIVETAR_SIZES, rivetar_configs, rivetar_work),
                                  "lobutar": (LOBUTAR_SIZES, lobutar_configs, lobutar_work),
                                  "tolanex": (COMPARE_SIZES, compare_configs, tolanex_work)}[first]
    out = {"compare": f"{first} beside llama at equal width, depth and (active) feed-forward size", "dtype": "bf16",
           "data": "synthetic: random weights, uniform random token ids", "peaks": pk, "sizes": {}}
    steps, warmup = min(args.steps, 200), max(args.warmup, 3)
    for name, z in sizes.items():
        if args.size not in ("all", name):
            continue
        if first == "bifatar":
            z = dict(z, layers=len(z["order"]), top=1, ff=z["llama_ff"], shared=0)      # the keys llama_work reads
        elif first == "rivetar":
            z = dict(z, layers=len(rivetar_runs(z)), top=1, ff=z["llama_ff"], shared=0)
        elif first == "lobutar":
            z = dict(z, layers=len(z["order"]), top=1, ff=z["llama_ff"], shared=0)
        res = {}
        for arch, cfg in zip((first, "llama"), configs(z)):
            tensors = dict(random_tensors(cfg, 0, torch.bfloat16, device="cuda:0"))
            spec = model_from_tensors(cfg, tensors, "bfloat16", "cuda:0")
            del tensors
            max_len = 1280 + warmup + steps + 64
            ec = EngineConfig(kv=KVManagerConfig(num_blocks=8 * (max_len // BLOCK_SIZE + 2) + 160, block_size=BLOCK_SIZE,
                                                 max_seq_len=max(max_len, PREFILL_TOKENS + 16), watermark_blocks=0),
                              sched=SchedulerConfig(max_num_seqs=8, max_batched_tokens=4096), dtype="bfloat16")
            dec = decode_run(spec, ec, COMPARE_VOCAB, 8, steps, warmup, 1280 - warmup - steps // 2)   # contexts of one graph bucket
            pre = prefill_times(spec, ec, COMPARE_VOCAB)
            fam = {k: {kk: {"calls": c, "ms": round(ms, 4)} for kk, (c, ms) in family_profile(spec, COMPARE_VOCAB, k).items()}
                   for k in ("prefill", "decode")}
            work = {"prefill": (first_work if arch == first else llama_work)(z, PREFILL_TOKENS, PREFILL_TOKENS, False),
                    "decode": (first_work if arch == first else llama_work)(z, 8, 1024, True)}
            res[arch] = {"decode_tokens_per_s": round(8 * steps * 1e3 / dec["dev_ms"], 1),
                         "decode_ms_per_step": round(dec["dev_ms"] / steps, 4),
                         "decode_e2e_tokens_per_s": round(8 * steps * 1e3 / dec["wall_ms"], 1),
                         "decode_graph_steps": dec["graph_steps"], "gpu_launches": int(dec["launches"]),
                         "prefill_tokens_per_s": round(PREFILL_TOKENS * 1e3 / pre[0], 1), "prefill_ms": round(pre[0], 3),
                         "prefill_e2e_ms": round(pre[1], 3), "families": fam, "work": work}
            del spec
            torch.cuda.empty_cache()
        out["sizes"][name] = dict(z, **res)
    print(json.dumps(out))
    return 0


def prefill_times(spec, ec, vocab, reps=3):
    """(device ms, end-to-end ms) of one prompt of PREFILL_TOKENS tokens in one step through the engine."""
    import torch
    from kvcm.engine.engine import DeviceTimer, Engine
    eng = Engine(spec, ec)
    g = torch.Generator().manual_seed(2)
    dev, wall = [], []
    for r in range(reps + 2):
        toks = torch.randint(3, vocab, (PREFILL_TOKENS,), generator=g).tolist()
        timer = DeviceTimer()
        eng.device_timer = timer
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.add_request(toks, max_new_tokens=1)
        info = eng.step()
        t1 = time.perf_counter()
        assert info.prefill_tokens == PREFILL_TOKENS and info.sampled == 1, info
        eng.take_finished()
        ms = timer.total_ms()
        eng.device_timer = None
        if r >= 2:
            dev.append(ms)
            wall.append((t1 - t0) * 1e3)
    del eng
    torch.cuda.empty_cache()
    return statistics.median(dev), statistics.median(wall)


def reference_main(args) -> int:
    """The same metric and shape through the unmodified reference (fp16, its own kvbench)."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ra
    if args.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a single-GPU engine"}))
        return 0
    steps, warmup, B = args.steps, max(args.warmup, 3), args.batch
    layers = MODEL["num_hidden_layers"]
    prompt_len = window_prompt_len(steps, warmup)
    kv_per_token = 2 * 2 * layers * MODEL["num_key_value_heads"] * MODEL["head_dim"]
    max_len = max(CONTEXT, prompt_len + warmup + steps + 64 + 16)
    pk = peaks()
    work = None
    try:
        ra.ensure_built()
        work = ra.make_workdir()
        wfile = os.path.join(work, "weights.bin")
        ra.write_weight_file(wfile, MODEL, seed=0)
        clocks = ClockSampler()
        clocks.start()
        main_run = ra.decode_run(wfile, B, prompt_len, steps, warmup, kv_per_token, max_len, work)
        clk = clocks.stop()
        pts, prefill = {}, None
        if not args.no_points:
            for b in (1, 64):
                r = ra.decode_run(wfile, b, prompt_len, steps, warmup, kv_per_token, max_len, work)
                pts[f"decode_b{b}"] = round(b * 1e3 / r["ms_per_step"], 1)
            prefill = ra.prefill_run(wfile, PREFILL_TOKENS, 7, work)
    except ra.ReferenceUnavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)}))
        return 0
    except subprocess.TimeoutExpired:
        print(json.dumps({"impl": "reference", "unavailable": "the reference's kvbench did not end in time"}))
        return 0
    finally:
        if work:
            import shutil
            shutil.rmtree(work, ignore_errors=True)
    H, I, V = MODEL["hidden_size"], MODEL["intermediate_size"], MODEL["vocab_size"]
    qkv = (MODEL["num_attention_heads"] + 2 * MODEL["num_key_value_heads"]) * MODEL["head_dim"]
    per_layer = qkv * H + H * H + 2 * I * H + H * I
    weight_bytes = 2 * (per_layer * layers + V * H + (2 * layers + 1) * H)
    ms = main_run["ms_per_step"]
    value = B * 1e3 / ms
    achieved = (weight_bytes + B * main_run["mean_ctx"] * kv_per_token) / (ms * 1e-3) / 1e9
    out = {
        "metric": "decode tokens/s (TinyLlama-1.1B shape, batch 8, 1,024-token prompts decoded towards 2,048)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / PUBLISHED[B], 2) if B in PUBLISHED else None,
        "dtype": "fp16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "impl": "reference",
        "config": {"model": "TinyLlama-1.1B shape (Llama dense decoder)", "layers": layers,
                   "layers_full": layers, "hidden": H, "heads": MODEL["num_attention_heads"],
                   "kv_heads": MODEL["num_key_value_heads"], "head_dim": MODEL["head_dim"], "ffn": I,
                   "vocab": V, "global_batch": B, "seq_len": CONTEXT, "prompt_len": prompt_len,
                   "mean_context": round(main_run["mean_ctx"], 1), "kv_block": BLOCK_SIZE,
                   "parallelism": "single GPU", "cuda_graphs": False, "gemm": "cuBLAS",
                   "l2": "inputs larger than L2 (2.2 GB of weights read per step)",
                   "peaks": pk["source"],
                   "timing": "host clock of the reference's own step log (schedule, copies, forward, synchronize)"},
        # The reference has one clock, around its whole step on the host: both figures are that one.
        "e2e": {"value": round(value, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": int(4 * (6 * B + B * ((max_len + BLOCK_SIZE - 1) // BLOCK_SIZE))),
                "d2h_bytes_per_step": 4 * B},
        "gpu_launches": 13 * layers + 4 + 2 * layers,   # src/model/llama.cpp:104-129, attention v2 adds its merge
        "clocks": clk,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]},
    }
    if pts:
        out["points"] = pts
    if prefill:
        flops = 2.0 * per_layer * layers * PREFILL_TOKENS + 2.0 * V * H \
            + 4.0 * MODEL["head_dim"] * MODEL["num_attention_heads"] * (PREFILL_TOKENS * (PREFILL_TOKENS + 1) / 2) * layers
        out["prefill"] = {"value": round(PREFILL_TOKENS * 1e3 / prefill, 1), "tokens": PREFILL_TOKENS,
                          "ms": round(prefill, 3),
                          "frac": round(flops / (prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=MODEL["num_hidden_layers"])
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64 and the prefill")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--gemm", default="auto", choices=["auto", "native", "library"],
                    help="bfloat16 products: 'auto' the fastest measured (this engine's kernels or the library), "
                         "'native' this engine's kernels only, 'library' the library wherever it can stand")
    ap.add_argument("--only", default="all", choices=["all", "prefill"],
                    help="'prefill': run only the 2,048-token prefill step and print its numbers (for profiling)")
    ap.add_argument("--compare", default="", choices=["", "tolanex", "bifatar", "rivetar", "lobutar"],
                    help="'tolanex' | 'bifatar' | 'rivetar' | 'lobutar': instead of the default workload, prefill and decode of that design beside "
                         "the Llama decoder at equal sizes, with device time per kernel family")
    ap.add_argument("--size", default="all", choices=["all"] + sorted(COMPARE_SIZES) + sorted(BIFATAR_SIZES) + sorted(RIVETAR_SIZES) + sorted(LOBUTAR_SIZES),
                    help="with --compare: one size only")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_main(args)
    if args.compare:
        return compare_main(args)
    if args.gpus != 1:
        print(f"bench.py: this engine is single-GPU by design; --gpus {args.gpus} is not supported "
              f"(run with --gpus 1)")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    if not torch.cuda.is_available():
        print("bench.py: no CUDA device", file=sys.stderr)
        return 1
    steps, warmup, layers = args.steps, args.warmup, args.layers
    # Requests admitted first already decode while later prompts are still being prefilled.
    prompt_len = window_prompt_len(steps, warmup)
    head = 64 * prompt_len // 4096 + 32
    max_len = max(CONTEXT, prompt_len + warmup + steps + head)
    pk = peaks()

    cfg, spec, ec = build_engine(layers, max(args.batch, 64 if not args.no_points else args.batch),
                                 max_len, graphs=not args.no_graphs)
    ec.gemm = args.gemm
    vocab = cfg.vocab_size
    m = model_bytes_and_flops(cfg, layers)
    if args.only == "prefill":
        ms, flops, wall = prefill_run(spec, ec, vocab, cfg, layers, reps=3)
        print(json.dumps({"prefill": {"value": round(PREFILL_TOKENS * 1e3 / ms, 1), "tokens": PREFILL_TOKENS,
                                      "ms": round(ms, 3), "layers": layers, "e2e_ms": round(wall, 3),
                                      "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}}))
        return 0

    main_run = decode_run(spec, ec, vocab, args.batch, steps, warmup, prompt_len, sample_clocks=True)
    B = args.batch
    ms_per_step = main_run["dev_ms"] / steps
    value = B * 1e3 / ms_per_step
    e2e_value = B * steps * 1e3 / main_run["wall_ms"]
    step_bytes = m["weight_bytes"] + B * main_run["mean_ctx"] * m["kv_bytes_per_token"]
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9

    out = {
        "metric": "decode tokens/s (TinyLlama-1.1B shape, batch 8, 1,024-token prompts decoded towards 2,048)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / PUBLISHED[B], 2) if B in PUBLISHED else None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "impl": "ours",
        "config": {"model": "TinyLlama-1.1B shape (Llama dense decoder)", "layers": layers,
                   "layers_full": MODEL["num_hidden_layers"], "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "ffn": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": B, "seq_len": CONTEXT, "prompt_len": prompt_len,
                   "mean_context": round(main_run["mean_ctx"], 1), "kv_block": BLOCK_SIZE,
                   "parallelism": "single GPU", "cuda_graphs": not args.no_graphs, "gemm": args.gemm,
                   "l2": "inputs larger than L2 (2.2 GB of weights read per step)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": int(main_run["h2d"]), "d2h_bytes_per_step": int(main_run["d2h"])},
        "gpu_launches": int(main_run["launches"]),
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4),
                     "of": pk["source"]},
    }
    if not args.no_points:
        pts = {}
        for b in (1, 64):
            r = decode_run(spec, ec, vocab, b, steps, warmup, prompt_len)
            pts[f"decode_b{b}"] = round(b * steps * 1e3 / r["dev_ms"], 1)
            # the same roofline fraction as above: bytes the step has to read over its time, of the copy rate
            need = m["weight_bytes"] + b * r["mean_ctx"] * m["kv_bytes_per_token"]
            pts[f"decode_b{b}_hbm_frac"] = round(need / (r["dev_ms"] / steps * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        out["points"] = pts
        ms, flops, wall = prefill_run(spec, ec, vocab, cfg, layers)
        out["prefill"] = {"value": round(PREFILL_TOKENS * 1e3 / ms, 1), "tokens": PREFILL_TOKENS,
                          "ms": round(ms, 3), "e2e_ms": round(wall, 3),
                          "e2e_value": round(PREFILL_TOKENS * 1e3 / wall, 1),
                          "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
