"""Rivetar configurations drawn at random (fixed seeds): odd widths, head, value and latent sizes (also sizes
the tensor-core kernels take only after padding), rotations from 2 dimensions to the whole (rotated part of a)
head, windows from 2 tokens up to longer than the sequence with none, few or many kept first tokens, every layer
order, layers without a feed-forward, decay ranks from 1, loops anywhere (also of one pass, and over all layers)
or none, a cap on the logits or none, page sizes 8 / 16 / 32.  Each model runs whole, in portions with single
tokens between them, and beside a second request, in float32 and bfloat16, against the plain implementation.

float32: every position within the float32 bound.  bfloat16: these models are not tuned to be well
conditioned, so single positions can move by much under 16-bit rounding; what is held is that the typical
position is within 6 % of the spread and at least 75 % are within 10 % (some draws run thirteen layer runs at a
width of 24): a size the kernels mishandle, a lost
key or a wrong state moves nearly every position by the order of the spread."""
import random

import pytest
import torch

import helpers
import plain_rivetar as P
import rivetar_models as RM
from test_gpu_rivetar import close

pytestmark = pytest.mark.gpu


def close_typical(got, ref, what):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert got.shape == ref.shape and torch.isfinite(got).all(), what
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    err = d.pow(2).mean(dim=-1).sqrt() / ref.std().item()
    assert err.median().item() <= 0.06 and (err <= 0.10).double().mean().item() >= 0.75, \
        f"{what}: median {err.median().item():.3f}, {int((err > 0.10).sum())} of {err.numel()} beyond 10 %"


def draw(seed: int) -> dict:
    r = random.Random(seed)
    layers = []
    for i in range(r.randint(1, 5)):
        kind = r.choice(["attention", "latent_attention", "gla"])
        if kind == "attention":
            kv = r.choice([1, 2, 3])
            dim = r.choice([6, 9, 16, 20, 32, 40, 64])
            m = RM.attn(kv * r.choice([1, 2, 4]), kv, dim, r.choice([6, 8, 16, 24, 34, 64]), round(r.uniform(0.05, 0.5), 3),
                        (r.choice([50.0, 10000.0, 1e6]), r.choice([d for d in (2, 4, 6, 8, 16, 20, 32, 64) if d <= dim])))
            if r.random() < 0.8:
                m["mask"] = {"size": r.choice([2, 3, 8, 15, 16, 17, 40, 64, 200])}
                if r.random() < 0.8:
                    m["mask"]["keep_first"] = r.choice([0, 1, 2, 4, 16, 17, 70])
        elif kind == "latent_attention":
            rot_dim = r.choice([2, 4, 6, 16, 32])
            m = RM.latent(r.choice([1, 2, 3, 5]), r.choice([3, 8, 16, 24, 33]), rot_dim, r.choice([5, 8, 16, 40]),
                          r.choice([7, 16, 24, 48, 60, 112]), r.choice([5, 8, 24, 33]), round(r.uniform(0.05, 0.5), 3),
                          (r.choice([20.0, 10000.0, 250000.0]), r.choice([d for d in (2, 4, 6, 16, 32) if d <= rot_dim])))
        else:
            m = RM.gla(r.choice([1, 2, 3, 4]), r.choice([3, 4, 9, 16, 33, 64, 100]), r.choice([5, 8, 24, 40]),
                       r.choice([1.0, 4.0, 16.0, 50.0]), r.choice([1, 3, 8, 12, 17]))
        mlp = RM.dense(r.choice([8, 20, 37, 64])) if r.random() < 0.7 else None
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    cfg = {"architecture": "Rivetar", "vocab": r.choice([61, 100, 257]), "width": r.choice([24, 40, 52, 66, 88, 130]),
           "norm": {"eps": r.choice([1e-6, 1e-5, 3e-4])}, "embedding": {"scale": r.choice([1.0, 0.5, 3.0, 11.0])}, "layers": layers}
    if r.random() < 0.6:
        cfg["logit_softcap"] = r.choice([5.0, 15.0, 30.0])
    if r.random() < 0.7:
        a = r.randrange(len(layers))
        cfg["loop"] = {"start": a, "stop": r.randint(a + 1, len(layers)), "times": r.choice([1, 2, 2, 3])}
    return cfg


@pytest.mark.parametrize("seed", range(12))
def test_random_configuration(seed, tmp_path):
    cfg = draw(seed)
    B = (8, 16, 32)[seed % 3]
    toks, other = helpers.random_tokens(75, cfg["vocab"], 500 + seed), helpers.random_tokens(41, cfg["vocab"], 900 + seed)
    for dtype in ("float32", "bfloat16"):
        folder = RM.write_model_from(cfg, 100 + seed, dtype, str(tmp_path / dtype))
        cfg_read, w = RM.read_model(folder)
        ref, ref2 = P.forward(cfg_read, w, toks), P.forward(cfg_read, w, other)
        r = helpers.Replayer(folder, dtype, 256, B, max_live=3)
        whole = r.step([dict(id="w", tokens=toks, want=list(range(75)))], end=["w"])
        check = (lambda g, rf, what: close(g, rf, dtype, what)) if dtype == "float32" else close_typical
        check(whole, ref, f"seed {seed} whole ({cfg})")
        outs, second, at, at2 = [], [], 0, 0
        for k in (1, 2, 30, 1, 17, 2, 1, 1, 20):
            entries = [dict(id="p", tokens=toks[at:at + k], want=list(range(k)))]
            k2 = min(5 if k > 1 else 1, len(other) - at2)
            if k2 > 0:
                entries.append(dict(id="q", tokens=other[at2:at2 + k2], want=list(range(k2))))
            out = r.step(entries)
            outs.append(out[:k])
            second.append(out[k:])
            at, at2 = at + k, at2 + max(k2, 0)
        assert at == 75
        check(torch.cat(outs), ref, f"seed {seed} in portions")
        check(torch.cat(second), ref2[:at2], f"seed {seed} second request")


def draw_larger(seed: int) -> dict:
    """Sizes of a small real model: widths of 128 to 512, heads of 32 to 128, cached latent rows of 72 to 384
    elements (beyond 256 the plain attention kernel serves them), three to eight layers."""
    r = random.Random(1000 + seed)
    layers = []
    for i in range(r.randint(3, 8)):
        kind = r.choice(["attention", "latent_attention", "latent_attention", "gla"])
        if kind == "attention":
            kv, dim = r.choice([1, 2, 4]), r.choice([32, 48, 64, 96, 128])
            m = RM.attn(kv * r.choice([1, 2, 4]), kv, dim, r.choice([32, 48, 64, 96, 128]), round(dim ** -0.5, 4),
                        (r.choice([10000.0, 20000.0, 500000.0]), r.choice([d for d in (16, 32, 48, 64, 96, 128) if d <= dim])))
            if r.random() < 0.9:
                m["mask"] = {"size": r.choice([16, 24, 50, 64, 72, 100, 128, 200]), "keep_first": r.choice([0, 1, 2, 4, 8])}
        elif kind == "latent_attention":
            rot, dim = r.choice([8, 16, 32, 64]), r.choice([32, 64, 96, 128])
            m = RM.latent(r.choice([2, 4, 6, 8]), dim, rot, r.choice([32, 48, 64, 128]), r.choice([64, 96, 128, 192, 256, 320]),
                          r.choice([64, 128, 192, 256]), round((dim + rot) ** -0.5, 4), (r.choice([10000.0, 250000.0]), rot))
        else:
            m = RM.gla(r.choice([1, 2, 4]), r.choice([32, 48, 64, 128]), r.choice([32, 64, 96]), r.choice([4.0, 16.0, 32.0]),
                       r.choice([8, 16, 32]))
        layers.append({"type": kind, "mixer": m, "mlp": RM.dense(r.choice([256, 512, 768, 1024])) if r.random() < 0.8 else None})
    cfg = {"architecture": "Rivetar", "vocab": r.choice([512, 1000, 2048]), "width": r.choice([128, 192, 320, 384, 512]),
           "norm": {"eps": r.choice([1e-6, 1e-5])}, "embedding": {"scale": r.choice([1.0, 2.0, 8.0])}, "layers": layers,
           "logit_softcap": r.choice([20.0, 50.0])}
    if r.random() < 0.85:
        a = r.randrange(len(layers))
        cfg["loop"] = {"start": a, "stop": r.randint(a + 1, len(layers)), "times": r.choice([1, 2, 2, 3])}
    return cfg


def spread_error(got, ref):
    d = got.double().cpu() - ref.double().cpu()
    d = d - d.mean(dim=-1, keepdim=True)
    return d.pow(2).mean(dim=-1).sqrt() / ref.double().std().item()


@pytest.mark.parametrize("seed", range(8))
def test_random_configuration_at_larger_sizes(seed, tmp_path):
    """Pages of 64, a prompt of 330 tokens whole and in portions cut at random beside a second request, float32:
    every position within 2e-4 of the logits' spread; bfloat16: the typical position within 3 %."""
    cfg = draw_larger(seed)
    n = 330
    toks, other = helpers.random_tokens(n, cfg["vocab"], 40 + seed), helpers.random_tokens(200, cfg["vocab"], 80 + seed)
    for dtype in ("float32", "bfloat16"):
        folder = RM.write_model_from(cfg, 300 + seed, dtype, str(tmp_path / dtype))
        cfg_read, w = RM.read_model(folder)
        ref, ref2 = P.forward(cfg_read, w, toks), P.forward(cfg_read, w, other)
        r = helpers.Replayer(folder, dtype, 768, 64, max_live=4)
        errs = [spread_error(r.step([dict(id="w", tokens=toks, want=list(range(n)))], end=["w"]), ref)]
        rnd, at, at2, outs, second = random.Random(seed), 0, 0, [], []
        while at < n:
            k = min(rnd.choice([1, 2, 3, 40, 64, 65, 100]) if at < 250 else 1, n - at)
            entries = [dict(id="p", tokens=toks[at:at + k], want=list(range(k)))]
            k2 = min(rnd.choice([1, 2, 17]), len(other) - at2)
            if k2 > 0:
                entries.append(dict(id="q", tokens=other[at2:at2 + k2], want=list(range(k2))))
            out = r.step(entries)
            outs.append(out[:k])
            second.append(out[k:])
            at, at2 = at + k, at2 + max(k2, 0)
        errs += [spread_error(torch.cat(outs), ref), spread_error(torch.cat(second), ref2[:at2])]
        for what, e in zip(("whole", "in portions", "second request"), errs):
            assert torch.isfinite(e).all(), f"seed {seed} {dtype} {what}: non-finite ({cfg})"
            if dtype == "float32":
                assert e.max().item() < 2e-4, f"seed {seed} float32 {what}: {e.max().item():.2e} at {int(e.argmax())} ({cfg})"
            else:
                assert e.median().item() < 0.03, f"seed {seed} bfloat16 {what}: median {e.median().item():.3f} ({cfg})"
