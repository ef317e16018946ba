"""Lobutar in the engine against the plain implementation (``plain_lobutar.py``, float64, whole sequences): every
way of cutting the work, every kind of layer alone, pages that are used again, keys far away, at page borders and at
a window's edge, the first tokens, long decoding, the new kernels alone, and greedy generation through the engine's
own entry point and scheduler.

float32 engine: every logit within 5e-4 of the plain logits' spread (the test models' output heads are scaled up so
that the logits spread over several units).  bfloat16 engine: per position, the root mean square of the difference
(mean taken off) is held against the spread of the plain logits: at most 5 % of the positions beyond 10 %, none
beyond 40 % (a wrong kernel path or a stale page moves most positions by the order of the spread itself; what one
lost key among hundreds does is the float32 engine's business).
"""
import itertools

import pytest
import torch

import helpers
import lobutar_models as LM
import plain_lobutar as P

pytestmark = pytest.mark.gpu

NAMES = ("lob-a", "lob-b", "lob-c")
LENGTHS = {"lob-a": [1, 9, 47, 130, 300], "lob-b": [3, 64, 150, 257], "lob-c": [2, 33, 190]}
CASES = [(n, d) for n in NAMES for d in ("float32", "bfloat16")]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[(name, dtype)] = LM.write_model(name, dtype, str(tmp_path_factory.mktemp(f"{name}_{dtype}")))
        return made[(name, dtype)]
    return get


@pytest.fixture(scope="module")
def oracle(folders):
    cache = {}

    def get(name, dtype, i):
        if (name, dtype, i) not in cache:
            cache[(name, dtype, i)] = LM.plain_logits(folders(name, dtype), tokens_of(name, i))
        return cache[(name, dtype, i)]
    return get


def tokens_of(name, i):
    return helpers.random_tokens(LENGTHS[name][i], LM.CONFIGS[name]["cfg"]["vocab"], 700 + i)


def replayer(folders, name, dtype, max_tokens, **kw):
    return helpers.Replayer(folders(name, dtype), dtype, max_tokens, LM.CONFIGS[name]["block_size"], **kw)


def close(got, ref, dtype, what):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    if dtype == "float32":
        worst, bound = (got - ref).abs().max().item(), 5e-4 * max(1.0, ref.std().item())
        assert worst <= bound, f"{what}: float32 logits differ by {worst:.3e} (bound {bound:.3e}) at {int((got - ref).abs().max(dim=-1).values.argmax())}"
        return
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    err = d.pow(2).mean(dim=-1).sqrt() / ref.std().item()
    over = int((err > 0.10).sum())
    assert over <= max(1, int(0.05 * err.numel())) and err.max().item() < 0.4, \
        f"{what}: {over} of {err.numel()} positions beyond 10 % of the spread (worst {err.max().item():.3f} at {int(err.argmax())})"


# ------------------------------------------------------------------------ ways of cutting the work

@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_requests(name, dtype, folders, oracle):
    r = replayer(folders, name, dtype, 320)
    for i, n in enumerate(LENGTHS[name]):
        toks = tokens_of(name, i)
        got = r.step([dict(id=f"r{i}", tokens=toks, want=list(range(n)))], end=[f"r{i}"])
        close(got, oracle(name, dtype, i), dtype, f"{name} whole request {i}")
    assert r.kv.blocks_in_use() == 0
    assert r.stray_writes() == []


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_against_token_by_token(name, dtype, folders, oracle):
    """The second request token by token from its first token on (the first tokens have fewer keys than a window
    holds); the longest mostly as one portion, then 60 single tokens (windows pass over decoded tokens)."""
    r = replayer(folders, name, dtype, 320)
    toks, ref = tokens_of(name, 1), oracle(name, dtype, 1)
    outs = [r.step([dict(id="x", tokens=[t], want=[0])]) for t in toks]
    close(torch.cat(outs), ref, dtype, f"{name} token by token")
    r.session.release("x")
    i = len(LENGTHS[name]) - 1
    toks, ref = tokens_of(name, i), oracle(name, dtype, i)
    head = len(toks) - 60
    outs = [r.step([dict(id="y", tokens=toks[:head], want=list(range(head)))])]
    outs += [r.step([dict(id="y", tokens=[t], want=[0])]) for t in toks[head:]]
    close(torch.cat(outs), ref, dtype, f"{name} prefill then 60 single tokens")


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_down_to_two_tokens(name, dtype, folders, oracle):
    r = replayer(folders, name, dtype, 320)
    sizes = itertools.cycle([7, 2, 13, 2, 1, 5, 31, 3, 2, 17, 64, 1, 1, 2])
    for i, n in enumerate(LENGTHS[name]):
        toks = tokens_of(name, i)
        outs, at = [], 0
        while at < n:
            k = min(next(sizes), n - at)
            outs.append(r.step([dict(id="p", tokens=toks[at:at + k], want=list(range(k)))]))
            at += k
        r.session.release("p")
        close(torch.cat(outs), oracle(name, dtype, i), dtype, f"{name} request {i} in portions")


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_requests_together_with_pages_used_again(name, dtype, folders, oracle):
    """Up to three live requests in a pool that cannot hold all requests at once: some bring a portion while others
    bring one token; a request that ends gives its pages to the next one."""
    B = LM.CONFIGS[name]["block_size"]
    lens = LENGTHS[name]
    todo = list(range(len(lens))) + [1, 0]                       # two of them a second time
    pool = helpers.roundup(max(lens), B) + 2 * helpers.roundup(sorted(lens)[-2], B)
    r = replayer(folders, name, dtype, pool, max_live=3)
    cuts = itertools.cycle([11, 1, 2, 29, 1, 1, 5, 64, 3, 1])
    live, got, step_no = {}, {}, 0
    while todo or live:
        held = sum(helpers.roundup(len(tokens_of(name, i)), B) for i, _ in live.values())
        while todo and len(live) < 3 and held + helpers.roundup(lens[todo[0]], B) <= pool:
            i = todo.pop(0)
            held += helpers.roundup(lens[i], B)
            live[f"q{step_no}_{i}"] = (i, 0)
            got[f"q{step_no}_{i}"] = []
        entries, ends = [], []
        for rid, (i, at) in list(live.items()):
            toks = tokens_of(name, i)
            k = min(next(cuts), len(toks) - at)
            entries.append(dict(id=rid, tokens=toks[at:at + k], want=list(range(k))))
            live[rid] = (i, at + k)
            if at + k == len(toks):
                ends.append(rid)
        out = r.step(entries, end=())
        row = 0
        for e in entries:
            got[e["id"]].append(out[row:row + len(e["tokens"])])
            row += len(e["tokens"])
        for rid in ends:
            r.session.release(rid)
            del live[rid]
        step_no += 1
    for rid, parts in got.items():
        i = int(rid.split("_")[1])
        close(torch.cat(parts), oracle(name, dtype, i), dtype, f"{name} request {rid} among others")
    assert r.kv.blocks_in_use() == 0
    assert len(set(r.pages_seen)) < len(r.pages_seen)            # pages were handed out more than once


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, folders, oracle):
    """A short prompt, then 260 tokens one by one: the pages grow across many borders and the window passes over
    decoded tokens (its pages are given back on the way)."""
    name = "lob-a"
    toks, ref = tokens_of(name, 4), oracle(name, dtype, 4)
    r = replayer(folders, name, dtype, 320)
    outs = [r.step([dict(id="d", tokens=toks[:40], want=list(range(40)))])]
    outs += [r.step([dict(id="d", tokens=[t], want=[0])]) for t in toks[40:]]
    close(torch.cat(outs), ref, dtype, "long decoding")


# ------------------------------------------------------------------------------ each layer kind alone

def one_layer_model(tmp_path, layers, dtype="float32", width=48, vocab=120, eps=3e-6, seed=5, streams=2, decisive=False):
    cfg = {"architecture": "Lobutar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "streams": streams,
           "layers": layers if isinstance(layers, list) else [layers]}
    return LM.write_model_from(cfg, seed, dtype, str(tmp_path / "m"), decisive=decisive)


_EXP = {"type": "attention", "mixer": LM.attn(2, 2, 8, 8, 0.4, 0.3, (100.0, 4)), "mlp": LM.moe(12, 3, 14, (3, 2), 1.3, 22)}
ALONE = [
    ("attention_gqa", {"type": "attention", "mixer": LM.attn(4, 2, 12, 20, 0.6, 0.5, (100.0, 6)), "mlp": None}, 2),
    ("attention_wide_values", {"type": "attention", "mixer": LM.attn(2, 1, 6, 40, 0.2, 0.3, (9.0, 6)), "mlp": LM.dense(40)}, 4),
    ("attention_unrotated_odd", {"type": "attention", "mixer": LM.attn(3, 3, 7, 9, 0.5, 0.4, None), "mlp": None}, 1),
    ("latent_window", {"type": "latent_attention", "mixer": LM.latent(3, 8, 12, 14, 20, 0.4, 50.0, 21), "mlp": None}, 3),
    ("latent_window_two", {"type": "latent_attention", "mixer": LM.latent(2, 10, 2, 6, 30, 0.3, 3.0, 2), "mlp": LM.dense(33)}, 2),
    ("latent_causal_long_rows", {"type": "latent_attention", "mixer": LM.latent(2, 24, 16, 20, 560, 0.05, 50.0), "mlp": None}, 2),
    ("experts_groups_shared", _EXP, 2),
    ("experts_all_chosen", {"type": "attention", "mixer": LM.attn(2, 2, 8, 8, 0.4, 0.3, (100.0, 4)), "mlp": LM.moe(3, 3, 9)}, 5),
    ("layer_run_three_times", [_EXP, dict(_EXP, weights_of=0), dict(_EXP, weights_of=0)], 3),
]


@pytest.mark.parametrize("layers,streams", [(l, s) for _, l, s in ALONE], ids=[n for n, _, _ in ALONE])
def test_one_layer_alone(tmp_path, layers, streams):
    """One layer of each kind (with every kind of feed-forward or none; one to five streams; the router as random
    weights make it) in float32: whole, and in portions with single tokens at the end."""
    folder = one_layer_model(tmp_path, layers, streams=streams)
    cfg, w = LM.read_model(folder)
    toks = helpers.random_tokens(90, 120, 77)
    ref = P.forward(cfg, w, toks)
    r = helpers.Replayer(folder, "float32", 128, 16)
    close(r.step([dict(id="a", tokens=toks, want=list(range(90)))], end=["a"]), ref, "float32", "whole")
    outs = [r.step([dict(id="b", tokens=toks[:2], want=[0, 1])]), r.step([dict(id="b", tokens=toks[2:41], want=list(range(39)))]),
            r.step([dict(id="b", tokens=toks[41:80], want=list(range(39)))])]
    outs += [r.step([dict(id="b", tokens=[t], want=[0])]) for t in toks[80:]]
    close(torch.cat(outs), ref, "float32", "portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", [
    {"type": "attention", "mixer": LM.attn(8, 2, 64, 128, 0.3, 0.07, (10000.0, 32)), "mlp": None},
    {"type": "attention", "mixer": LM.attn(4, 4, 32, 64, 0.5, 0.12, (10000.0, 32)), "mlp": LM.dense(512)},
    {"type": "attention", "mixer": LM.attn(6, 1, 128, 192, 0.7, 0.05, (250000.0, 64)), "mlp": None},
    {"type": "latent_attention", "mixer": LM.latent(8, 64, 32, 64, 96, 0.07, 10000.0, 100), "mlp": LM.moe(8, 2, 128, (2, 1), 1.5, 256)},
    {"type": "latent_attention", "mixer": LM.latent(4, 96, 64, 128, 192, 0.05, 250000.0, 300), "mlp": None},
], ids=["diff64x2_gqa", "diff32x2_ff", "diff128x2", "latent128_window_experts", "latent256_window"])
def test_mixers_at_the_sizes_of_the_fast_kernels(tmp_path, layer, dtype):
    """Head sizes that take the tensor-core attention kernels and experts that take the tensor-core products, in a
    prompt of three portions and 70 decoded tokens, beside a second request."""
    folder = one_layer_model(tmp_path, layer, dtype, width=256, vocab=200, decisive=True)
    cfg, w = LM.read_model(folder)
    toks, other = helpers.random_tokens(420, 200, 3), helpers.random_tokens(150, 200, 4)
    ref, ref2 = P.forward(cfg, w, toks), P.forward(cfg, w, other)
    r = helpers.Replayer(folder, dtype, 640, 16)
    outs = [r.step([dict(id="a", tokens=toks[:200], want=list(range(200)))]),
            r.step([dict(id="a", tokens=toks[200:203], want=[0, 1, 2]), dict(id="b", tokens=other[:100], want=list(range(100)))])]
    o2 = [outs[1][3:]]
    outs[1] = outs[1][:3]
    outs.append(r.step([dict(id="a", tokens=toks[203:350], want=list(range(147)))]))
    for k, t in enumerate(toks[350:]):
        e = [dict(id="a", tokens=[t], want=[0])]
        if k < 50:
            e.append(dict(id="b", tokens=[other[100 + k]], want=[0]))
        out = r.step(e)
        outs.append(out[:1])
        if k < 50:
            o2.append(out[1:])
    close(torch.cat(outs), ref, dtype, "first request")
    close(torch.cat(o2), ref2[:len(torch.cat(o2))], dtype, "second request")


# ------------------------------------------------------------ one key that carries all the weight

D_PLANT, PLANTED = 48, 119


def plant(tmp_path, dtype, kind, window, which_map):
    """A one-layer model in which every query points at the key of ONE token (id 119, used once per prompt) and all
    other scores are near zero.  The token's row of the table lies along coordinate 0, every other token has a common
    component along coordinate 1 and nothing along 0; keys read coordinate 0 and queries coordinate 1, in head
    dimensions that the rotation leaves alone (differential attention: in ``which_map`` only, the other map's scores
    stay flat).  Losing the key, or seeing it one position too long, changes the logits completely."""
    D = D_PLANT
    if kind == "attention":
        H, G, dk, dv = 2, 1, 16, 12
        layer = {"type": "attention", "mixer": LM.attn(H, G, dk, dv, 0.3, 0.1, (100.0, 8)), "mlp": None}
    else:
        H, dn, dr, dv, R = 2, 8, 4, 12, 24
        layer = {"type": "latent_attention", "mixer": LM.latent(H, dn, dr, dv, R, 0.7, 100.0, window), "mlp": None}
    folder = one_layer_model(tmp_path, layer, dtype, width=D)
    cfg, w = LM.read_model(folder)
    g = torch.Generator().manual_seed(9)
    w["embed"] = torch.randn(120, D, generator=g, dtype=torch.float64) * 0.3
    w["embed"][:, :2] = 0
    w["embed"][:, 1] = 2.0
    w["embed"][PLANTED] = 0
    w["embed"][PLANTED, 0] = 6.0
    w["l0.norm1"] = torch.ones(D, dtype=torch.float64)
    p = "l0.mix."
    if kind == "attention":
        wk = torch.randn(G * 2 * dk, D, generator=g, dtype=torch.float64) * 0.02
        wk[:, :2] = 0
        lo = which_map * dk + 12                     # dimensions 12..15 of the chosen map: not rotated
        wk[lo:lo + 4] = 0                            # no other token's key reaches into them ...
        wk[lo:lo + 4, 0] = 1.0                       # ... they hold the planted token's key
        wq = torch.zeros(H * 2 * dk, D, dtype=torch.float64)
        for h in range(H):
            at = (h * 2 + which_map) * dk + 12
            wq[at:at + 4, 1] = 1.0                   # every query: the same dimensions of the same map
        w[p + "q"], w[p + "k"] = wq, wk
        w[p + "q.b"], w[p + "k.b"] = torch.zeros(H * 2 * dk, dtype=torch.float64), torch.zeros(G * 2 * dk, dtype=torch.float64)
    else:
        wdkv = torch.randn(R + dr, D, generator=g, dtype=torch.float64) * 0.05
        wdkv[:, :2] = 0
        wdkv[0] = 0
        wdkv[0, 0] = 1.0                             # latent element 0: the planted token only
        wq = torch.zeros(H * (dn + dr), D, dtype=torch.float64)
        wuk = torch.randn(H * dn, R, generator=g, dtype=torch.float64) * 0.02
        for h in range(H):
            wq[h * (dn + dr), 1] = 1.0               # element 0 of every head's unrotated query: the common component
            wuk[h * dn] = 0
            wuk[h * dn, 0] = 1.0                     # element 0 of every head's unrotated key: the latent's element 0
        w[p + "dkv"], w[p + "q"], w[p + "uk"] = wdkv, wq, wuk
        w[p + "dkv.norm"] = torch.ones(R, dtype=torch.float64)
        w[p + "sink"] = torch.tensor([0.5, -1.0], dtype=torch.float64)
    LM.save_weights(folder, w, dtype)
    return folder


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind,window,which_map", [("attention", 0, 0), ("attention", 0, 1), ("latent_attention", 40, 0),
                                                   ("latent_attention", 33, 0), ("latent_attention", 0, 0)])
def test_one_key_that_stands_out(tmp_path, dtype, kind, window, which_map):
    """The planted key is tried as first key, just before, at and behind page borders, and far back; the asking
    positions are in a prompt's portion and decoded alone.  With a window the positions just inside it (distance
    window - 1) and just outside (distance window) are among them; the check that the plant works compares exactly
    these positions in the plain implementation."""
    folder = plant(tmp_path, dtype, kind, window, which_map)
    cfg, w = LM.read_model(folder)
    n, head = 200, 120
    for far in (0, 1, 15, 16, 17, 31, 32, 79, 81, 100, 150):
        toks = helpers.random_tokens(n, PLANTED, 40 + far)
        toks[far] = PLANTED
        ref = P.forward(cfg, w, toks)
        r = helpers.Replayer(folder, dtype, 256, 16)
        outs = [r.step([dict(id="f", tokens=toks[:far + 1], want=list(range(far + 1)))])]
        if far + 1 < head:
            outs.append(r.step([dict(id="f", tokens=toks[far + 1:head], want=list(range(head - far - 1)))]))
        outs += [r.step([dict(id="f", tokens=[t], want=[0])]) for t in toks[max(head, far + 1):]]
        close(torch.cat(outs), ref, dtype, f"planted key at {far}")
        spread = ref.std().item()
        toks2 = list(toks)
        toks2[far] = 5
        without = P.forward(cfg, w, toks2)
        last_in = n - 1 if not window else min(n - 1, far + window - 1)
        if last_in > far:                         # the key is seen up to here and carries the weight
            assert (without[last_in] - ref[last_in]).abs().max().item() > 0.5 * spread
        if window and far + window < n:           # and not one position later
            assert (without[far + window] - ref[far + window]).abs().max().item() < 1e-6 * max(1.0, spread)


# --------------------------------------------------------------------------------- kernels alone

def test_stream_kernel_writes_reads_and_gathers():
    """The kernel over the residual streams against float32 PyTorch: write only, read only, both, with a bias, with
    gathered rows, for widths that take the 16-byte form and widths that do not, one to nine streams."""
    from kvcm.kernels import library as K
    g = torch.Generator(device="cuda").manual_seed(1)
    for S, D, T in ((1, 40, 5), (2, 256, 33), (3, 72, 17), (4, 1000, 9), (9, 30, 4)):
        x = torch.randn(T, S, D, device="cuda", generator=g)
        y = torch.randn(T, D, device="cuda", generator=g)
        bias = torch.randn(D, device="cuda", generator=g)
        mix, outw, inw = (torch.randn(s, device="cuda", generator=g) for s in ((S, S), (S,), (S,)))
        w = torch.randn(D, device="cuda", generator=g)
        new = torch.einsum("sr,tsd->trd", mix.double(), x.double()) + outw.double()[None, :, None] * (y + bias).double()[:, None, :]
        u = torch.einsum("s,tsd->td", inw.double(), new)
        h_ref = w.double() * u / torch.sqrt((u * u).mean(-1, keepdim=True) + 1e-5)
        for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 1.5e-2)):
            xa, h = x.clone(), torch.empty(T, D, dtype=dt, device="cuda")
            K.hc_step(xa, y, bias, mix, outw, inw, w, h, 1e-5)
            assert torch.allclose(xa.double(), new, atol=2e-5 * new.abs().max().item())
            assert torch.allclose(h.double(), h_ref, atol=tol * h_ref.abs().max().item())
            xb = x.clone()                                         # the two halves as two launches give the same streams
            K.hc_step(xb, y, bias, mix, outw, None, None, None, 0.0)
            assert torch.equal(xb, xa)
            h2 = torch.empty_like(h)
            K.hc_step(xb, None, None, None, None, inw, w, h2, 1e-5)
            assert torch.equal(h2, h) and torch.equal(xb, xa)
            rows = torch.tensor([T - 1, 0], dtype=torch.int32, device="cuda")
            xc, h3 = x.clone(), torch.empty(2, D, dtype=dt, device="cuda")
            K.hc_step(xc, y, bias, mix, outw, inw, w, h3, 1e-5, rows)
            assert torch.equal(h3, h[[T - 1, 0]])
        e = torch.empty(T, S, D, device="cuda")
        table = torch.randn(50, D, device="cuda", generator=g).to(torch.bfloat16)
        ids = torch.randint(0, 50, (T,), device="cuda", generator=g).to(torch.int32)
        K.embed_streams(ids, table, e)
        assert torch.equal(e, table[ids.long()].float()[:, None, :].expand(T, S, D))


def test_combining_two_maps_and_gating():
    from kvcm.kernels import library as K
    g = torch.Generator(device="cuda").manual_seed(2)
    T, H, dv, HD = 19, 3, 20, 32
    a = torch.randn(T, 2 * H, HD, device="cuda", generator=g)
    gate = torch.randn(T, H + 5, device="cuda", generator=g)[:, 2:2 + H]          # a view with a row stride
    lam = torch.tensor([0.73], device="cuda")
    o = a[:, 0::2, :dv].double() - 0.73 * a[:, 1::2, :dv].double()
    ref = o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-4) * 0.6 * torch.sigmoid(gate.double())[:, :, None]
    out = torch.empty(T, H * dv, device="cuda")
    K.diff_combine(a, gate, lam, out, H, dv, 1e-4, 0.6)
    assert torch.allclose(out.double().view(T, H, dv), ref, atol=1e-5)
    ab = a.to(torch.bfloat16)
    outb = torch.empty(T, H * dv, device="cuda", dtype=torch.bfloat16)
    K.diff_combine(ab, gate, lam, outb, H, dv, 1e-4, 0.6)
    ob = ab[:, 0::2, :dv].double() - 0.73 * ab[:, 1::2, :dv].double()
    refb = ob / torch.sqrt((ob * ob).mean(-1, keepdim=True) + 1e-4) * 0.6 * torch.sigmoid(gate.double())[:, :, None]
    assert torch.allclose(outb.double().view(T, H, dv), refb, atol=2e-2)
    x = torch.randn(T, 37, device="cuda", generator=g)
    gl = torch.randn(T, 50, device="cuda", generator=g)[:, 13:]
    y = torch.empty_like(x)
    K.gate_mul(x, gl, y)
    assert torch.allclose(y, x * torch.sigmoid(gl), atol=1e-6)


@pytest.mark.parametrize("E,groups,top", [(16, (2, 1), 3), (12, (4, 2), 4), (7, None, 2), (64, (8, 3), 6), (4, (2, 2), 1)])
def test_router_kernel_with_sigmoid_scores_and_corrections(E, groups, top):
    """The router kernel against the plain router on random rows, with corrections large enough to make choice
    scores negative and to change who is chosen; weights are the uncorrected scores."""
    from kvcm.kernels import library as K
    g = torch.Generator().manual_seed(E)
    T, D = 300, 24
    h = torch.randn(T, D, generator=g)
    w = {"router": torch.randn(E, D, generator=g).double(), "correction": (torch.randn(E, generator=g) * 1.5 - 1.0).double()}
    r = {"experts": E, "top": top, "scale": 1.7}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    idx_ref, wt_ref = P.route(h.double(), w, r)
    idx = torch.empty(T, top, dtype=torch.int32, device="cuda")
    wt = torch.empty(T, top, dtype=torch.float32, device="cuda")
    G, keep = groups or (1, 1)
    K.moe_route(h.cuda(), w["router"].float().cuda(), E, G, keep, top, 1.7, idx, wt, None, "sigmoid", w["correction"].float().cuda(), 2)
    got = {(t, int(e)): float(x) for t in range(T) for e, x in zip(idx[t].tolist(), wt[t].tolist())}
    want = {(t, int(e)): float(x) for t in range(T) for e, x in zip(idx_ref[t].tolist(), wt_ref[t].tolist())}
    assert set(got) == set(want)
    assert max(abs(got[k] - want[k]) for k in want) < 1e-5
    without = torch.empty_like(idx)
    K.moe_route(h.cuda(), w["router"].float().cuda(), E, G, keep, top, 1.7, without, wt, None, "sigmoid", None, 2)
    assert not torch.equal(without.sort(-1).values, idx.sort(-1).values)          # the corrections did change choices


def test_layers_with_and_without_the_fused_stream_kernel(folders, oracle):
    name = "lob-a"
    toks = tokens_of(name, 2)
    a = replayer(folders, name, "float32", 64).step([dict(id="a", tokens=toks, want=list(range(len(toks))))])
    b = replayer(folders, name, "float32", 64, options={"fuse": False}).step([dict(id="a", tokens=toks, want=list(range(len(toks))))])
    assert torch.equal(a, b)
    close(a, oracle(name, "float32", 2), "float32", "fused")


# ------------------------------------------------------- the engine's own entry point and scheduler

@pytest.mark.parametrize("name", ["lob-a", "lob-c"])
def test_greedy_generation_through_the_engine(name, folders):
    """Scheduler with chunked prefill and few sequences at a time; every generated token must be the plain
    implementation's choice given the tokens before it (ties within 2e-4 allowed)."""
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    folder = folders(name, "float32")
    cfg, w = LM.read_model(folder)
    B = LM.CONFIGS[name]["block_size"]
    prompts = [helpers.random_tokens(n, cfg["vocab"], 70 + i) for i, n in enumerate([21, 4, 50, 13, 1, 33])]

    def run(graphs):
        ec = EngineConfig(kv=KVManagerConfig(num_blocks=256 // B, block_size=B, max_seq_len=96, watermark_blocks=0),
                          sched=SchedulerConfig(max_num_seqs=3, max_batched_tokens=24), dtype="float32", cuda_graphs=graphs)
        eng = kvcm.Engine.from_folder(folder, ec)
        return eng, kvcm.generate(eng, prompts, 20)

    eng, outs = run(True)
    assert eng.graphs is not None and eng.graphs.replays > 10         # decode steps were replayed from CUDA graphs
    for p, o in zip(prompts, outs):
        assert len(o) == 20
        logits = P.forward(cfg, w, list(p) + list(o))
        for k, tok in enumerate(o):
            row = logits[len(p) - 1 + k]
            assert row.max().item() - row[tok].item() <= 2e-4, (len(p), k, tok, int(row.argmax()))
    assert eng.kv.blocks_in_use(0) == 0
    eng2, outs2 = run(False)
    assert eng2.graphs is None and outs2 == outs


def test_generation_in_bfloat16_with_eviction(folders):
    """So few pages that running requests are evicted and computed again from their first token.  With room for all
    and without, every generated token is the plain implementation's choice given the tokens before it, or within
    the bfloat16 engine's rounding of it."""
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    folder = folders("lob-a", "bfloat16")
    cfg, w = LM.read_model(folder)
    prompts = [helpers.random_tokens(n, 211, 90 + i) for i, n in enumerate([30, 44, 25, 38])]

    def run(blocks):
        ec = EngineConfig(kv=KVManagerConfig(num_blocks=blocks, block_size=16, max_seq_len=96, watermark_blocks=0),
                          sched=SchedulerConfig(max_num_seqs=4, max_batched_tokens=64), dtype="bfloat16")
        eng = kvcm.Engine.from_folder(folder, ec)
        outs = kvcm.generate(eng, prompts, 30)
        return eng, outs

    roomy, outs = run(64)
    tight, outs2 = run(11)
    assert all(len(o) == 30 for o in outs + outs2)
    assert tight.sched.counters().preemptions > 0 and roomy.sched.counters().preemptions == 0
    for p, o in list(zip(prompts, outs)) + list(zip(prompts, outs2)):
        logits = P.forward(cfg, w, list(p) + list(o))
        tol = 0.15 * logits.std().item()
        for k, tok in enumerate(o):
            row = logits[len(p) - 1 + k]
            assert row.max().item() - row[tok].item() <= tol, (len(p), k, tok, int(row.argmax()))


def test_trace_tool_on_a_model_folder(tmp_path, folders, oracle):
    name, dtype = "lob-b", "float32"
    toks, ref = tokens_of(name, 2), oracle(name, dtype, 2)
    other = tokens_of(name, 1)
    steps = [dict(step=0, entries=[dict(id="a", tokens=toks[:70], want=[0, 69])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=toks[70:72], want=[1]), dict(id="b", tokens=other, want=[63])], end=["b"]),
             dict(step=2, entries=[dict(id="a", tokens=toks[72:], want=[len(toks) - 73])], end=["a"])]
    out = helpers.run_trace_tool(folders(name, dtype), dtype, steps, 512, str(tmp_path / "out"), vocab_key="vocab")
    got = torch.cat([torch.from_numpy(out[0]), torch.from_numpy(out[1][:1]), torch.from_numpy(out[2])])
    close(got, ref[[0, 69, 71, len(toks) - 1]], dtype, "trace tool")
    close(torch.from_numpy(out[1][1:]), oracle(name, dtype, 1)[[63]], dtype, "trace tool, second request")
