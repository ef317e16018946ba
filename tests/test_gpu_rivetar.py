"""Rivetar in the engine against the plain implementation (``plain_rivetar.py``, float64, whole
sequences): every way of cutting the work, every kind of layer alone, pages and state slots that are
used again, keys far away, at page borders, at a window's edge and among the kept first tokens, long
decoding, and greedy generation through the engine's own entry point and scheduler.

float32 engine: every logit within 5e-4 of the plain logits' spread (the test models' output heads are scaled up
so that the logits spread over several units; float32 rounding through nine layer runs, their softmaxes and
the recurrence reaches about 5e-5 of the spread, one lost key among hundreds about 3e-3).
bfloat16 engine: per position, the root mean square of the difference (mean taken off) is held
against the spread of the plain logits.  Unit roundoff 2^-9, some dozens of roundings on the way to a
logit, and norms on the sublayers' outputs that keep a sublayer's relative error whatever its size: 2 to 4 %
of the spread through nine layer runs at a width of 72, with single badly conditioned positions at 15 %
(the same positions however the work is cut); held: at most 5 % of the positions beyond 10 %, none beyond
40 % (a wrong kernel path, a wrong state or a stale page moves most positions by the order of the spread
itself; what one lost key among hundreds does is the float32 engine's business).
"""
import itertools
import json

import pytest
import torch

import helpers
import plain_rivetar as P
import rivetar_models as RM

pytestmark = pytest.mark.gpu

NAMES = ("riv-a", "riv-b", "riv-c")
LENGTHS = {"riv-a": [1, 9, 47, 130, 300], "riv-b": [3, 64, 150, 257], "riv-c": [2, 33, 190]}
CASES = [(n, d) for n in NAMES for d in ("float32", "bfloat16")]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[(name, dtype)] = RM.write_model(name, dtype, str(tmp_path_factory.mktemp(f"{name}_{dtype}")))
        return made[(name, dtype)]
    return get


@pytest.fixture(scope="module")
def oracle(folders):
    cache = {}

    def get(name, dtype, i):
        if (name, dtype, i) not in cache:
            cache[(name, dtype, i)] = RM.plain_logits(folders(name, dtype), tokens_of(name, i))
        return cache[(name, dtype, i)]
    return get


def tokens_of(name, i):
    return helpers.random_tokens(LENGTHS[name][i], RM.CONFIGS[name]["cfg"]["vocab"], 600 + i)


def replayer(folders, name, dtype, max_tokens, **kw):
    return helpers.Replayer(folders(name, dtype), dtype, max_tokens, RM.CONFIGS[name]["block_size"], **kw)


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
    assert r.kv.blocks_in_use() == 0 and r.slots.num_taken() == 0
    assert r.stray_writes() == []


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_against_token_by_token(name, dtype, folders, oracle):
    """The second request token by token from its first token on (the states start at zero, the first tokens have
    fewer keys than a window holds and are the ones a window keeps); the longest mostly as one portion, then
    60 single tokens (windows pass over decoded tokens)."""
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
def test_unequal_requests_together_with_pages_and_slots_used_again(name, dtype, folders, oracle):
    """Up to three live requests in a pool that cannot hold all requests at once and with three state slots: some
    requests bring a portion while others bring one token; a request that ends gives its pages and its slot to
    the next one, which must start from zero state."""
    B = RM.CONFIGS[name]["block_size"]
    lens = LENGTHS[name]
    todo = list(range(len(lens))) + [1, 0]                       # two of them a second time
    pool = helpers.roundup(max(lens), B) + 2 * helpers.roundup(sorted(lens)[-2], B)
    r = replayer(folders, name, dtype, pool, max_live=3)
    cuts = itertools.cycle([11, 1, 2, 29, 1, 1, 5, 64, 3, 1])
    live, got, step_no = {}, {}, 0
    slots_seen = []
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
        slots_seen += [r.live[e["id"]].state_slot for e in entries]
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
    assert set(slots_seen) <= {0, 1, 2} and r.slots.num_taken() == 0 and r.kv.blocks_in_use() == 0
    assert len(set(r.pages_seen)) < len(r.pages_seen)            # pages were handed out more than once


# ------------------------------------------------------------------------------ each layer kind alone

def one_layer_model(tmp_path, layer, dtype="float32", width=48, vocab=120, eps=3e-6, seed=5, **top):
    cfg = {"architecture": "Rivetar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": 1.7},
           "layers": [layer], **top}
    return RM.write_model_from(cfg, seed, dtype, str(tmp_path / "m"))


ALONE = [
    ("attention_window_keep", {"type": "attention", "mixer": RM.attn(4, 2, 12, 20, 0.5, (100.0, 6), 21, 4), "mlp": None}, {}),
    ("attention_causal_ff", {"type": "attention", "mixer": RM.attn(2, 1, 16, 8, 0.3, (9.0, 16)), "mlp": RM.dense(40)}, {}),
    ("attention_window_only", {"type": "attention", "mixer": RM.attn(3, 3, 10, 14, 0.4, (1000.0, 2), 17), "mlp": None}, {}),
    ("gla", {"type": "gla", "mixer": RM.gla(4, 6, 10, 4.0, 7), "mlp": None}, {}),
    ("gla_slow_decay_ff", {"type": "gla", "mixer": RM.gla(3, 36, 8, 64.0, 2), "mlp": RM.dense(16)}, {}),
    ("latent", {"type": "latent_attention", "mixer": RM.latent(3, 8, 12, 14, 20, 9, 0.4, (50.0, 8)), "mlp": None}, {}),
    ("latent_long_rows", {"type": "latent_attention", "mixer": RM.latent(2, 24, 16, 20, 560, 40, 0.05, (50.0, 16)), "mlp": None}, {}),
    ("gla_long_keys", {"type": "gla", "mixer": RM.gla(2, 200, 24, 8.0, 4), "mlp": None}, {}),
    ("latent_ff_looped", {"type": "latent_attention", "mixer": RM.latent(2, 10, 2, 6, 30, 12, 0.3, (3.0, 2)),
                          "mlp": RM.dense(33)}, {"loop": {"start": 0, "stop": 1, "times": 3}, "logit_softcap": 11.0}),
]


@pytest.mark.parametrize("layer,top", [(l, t) for _, l, t in ALONE], ids=[n for n, _, _ in ALONE])
def test_one_layer_alone(tmp_path, layer, top):
    """One layer of each kind (and the feed-forward with it or without; once as a loop of three passes; once with a
    cached latent row and once with keys longer than any tensor-core kernel takes) in float32: whole, and in
    portions with single tokens at the end."""
    folder = one_layer_model(tmp_path, layer, **top)
    cfg, w = RM.read_model(folder)
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
    {"type": "attention", "mixer": RM.attn(8, 2, 128, 128, 0.05, (10000.0, 64), 100, 7), "mlp": None},
    {"type": "attention", "mixer": RM.attn(8, 2, 128, 128, 0.05, (10000.0, 128), 100), "mlp": None},
    {"type": "attention", "mixer": RM.attn(4, 4, 64, 48, 0.08, (10000.0, 64), 300, 70), "mlp": None},
    {"type": "attention", "mixer": RM.attn(20, 1, 32, 32, 0.2, (10000.0, 16)), "mlp": None},
    {"type": "gla", "mixer": RM.gla(4, 128, 128, 16.0, 16), "mlp": None},
    {"type": "latent_attention", "mixer": RM.latent(8, 64, 32, 64, 96, 96, 0.07, (10000.0, 32)), "mlp": RM.dense(512)},
    {"type": "latent_attention", "mixer": RM.latent(4, 96, 64, 128, 192, 160, 0.05, (250000.0, 64)), "mlp": None},
], ids=["attn128_keep", "attn128_window", "attn64_48_keep70", "attn20heads", "gla128", "latent128", "latent256"])
def test_mixers_at_the_sizes_of_the_fast_kernels(tmp_path, layer, dtype):
    """Head and state sizes that take the tensor-core attention kernels and the wide forms of the recurrence
    kernel, in a prompt of three portions and 70 decoded tokens, beside a second request.  (A request's first
    position is left out for the gla layer in bfloat16: its state is k v^T there, the head's output (q.k) v, and
    the norm over it keeps only the sign of q.k, which rounding decides when q.k is near zero.)"""
    folder = one_layer_model(tmp_path, layer, dtype, width=256, vocab=200)
    skip = 1 if layer["type"] == "gla" and dtype == "bfloat16" else 0
    cfg, w = RM.read_model(folder)
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
    close(torch.cat(outs)[skip:], ref[skip:], dtype, "first request")
    close(torch.cat(o2)[skip:], ref2[skip:len(torch.cat(o2))], dtype, "second request")


# ------------------------------------------------------------ one key that carries all the weight

D_PLANT, PLANTED = 48, 119


def plant(tmp_path, dtype, kind, window, keep):
    """A one-layer model in which every query points at the key of ONE token (id 119, used once per prompt) and
    all other scores are near zero.  The token's row of the table lies along coordinate 0, every other token has a
    common component along coordinate 1 and nothing along 0; keys read coordinate 0 and queries coordinate 1, in
    head dimensions that the rotation leaves alone.  Losing the key, or seeing it one position too long, changes
    the logits completely; so does a value that is not turned back by the reader's own position."""
    D = D_PLANT
    if kind == "attention":
        H, G, dk, dv = 2, 1, 16, 12
        layer = {"type": "attention", "mixer": RM.attn(H, G, dk, dv, 0.1, (100.0, 8), window, keep), "mlp": None}
    else:
        H, dn, dr, dv, R, qr = 2, 8, 4, 12, 24, 16
        layer = {"type": "latent_attention", "mixer": RM.latent(H, dn, dr, dv, R, qr, 0.7, (100.0, 4)), "mlp": None}
    folder = one_layer_model(tmp_path, layer, dtype, width=D)
    cfg, w = RM.read_model(folder)
    g = torch.Generator().manual_seed(9)
    w["embed"] = torch.randn(120, D, generator=g, dtype=torch.float64) * 0.3
    w["embed"][:, :2] = 0
    w["embed"][:, 1] = 2.0
    w["embed"][PLANTED] = 0
    w["embed"][PLANTED, 0] = 6.0
    w["l0.norm1"] = torch.zeros(D, dtype=torch.float64)
    p = "l0.mix."
    if kind == "attention":
        wk = torch.randn(G * dk, D, generator=g, dtype=torch.float64) * 0.02
        wk[:, :2] = 0
        wk[12:16] = 0                                # no other token's key reaches into dimensions 12..15 (not rotated) ...
        wk[12:16, 0] = 1.0                           # ... which hold the planted token's key
        wq = torch.zeros(H * dk, D, dtype=torch.float64)
        for h in range(H):
            wq[h * dk + 12:h * dk + 16, 1] = 1.0     # every query: the same dimensions
        w[p + "q"], w[p + "k"] = wq, wk
        w[p + "sink"] = torch.tensor([0.5, -1.0], dtype=torch.float64)
    else:
        wdkv = torch.randn(R + dr, D, generator=g, dtype=torch.float64) * 0.05
        wdkv[:, :2] = 0
        wdkv[0] = 0
        wdkv[0, 0] = 1.0                             # latent element 0: the planted token only
        wdq = torch.randn(qr, D, generator=g, dtype=torch.float64) * 0.01
        wdq[:, :2] = 0
        wdq[0, 1] = 1.0                              # the query latent's element 0: the common component
        wuq = torch.zeros(H * (dn + dr), qr, dtype=torch.float64)
        wuk = torch.randn(H * dn, R, generator=g, dtype=torch.float64) * 0.02
        for h in range(H):
            wuq[h * (dn + dr), 0] = 1.0              # element 0 of every head's unrotated query
            wuk[h * dn] = 0
            wuk[h * dn, 0] = 1.0                     # element 0 of every head's unrotated key
        w[p + "dkv"], w[p + "dq"], w[p + "uq"], w[p + "uk"] = wdkv, wdq, wuq, wuk
        w[p + "dq.norm"] = torch.ones(qr, dtype=torch.float64)
        w[p + "dkv.norm"] = torch.ones(R, dtype=torch.float64)
    RM.save_weights(folder, w, dtype)
    return folder


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind,window,keep", [("attention", 40, 3), ("attention", 33, 17), ("attention", 0, None),
                                              ("latent_attention", 0, None)])
def test_one_key_that_stands_out(tmp_path, dtype, kind, window, keep):
    """The planted key is tried as first key, as the last kept and the first not kept token, just before, at and
    behind page borders, and far back; the asking positions are in a prompt's portion and decoded alone.  With a
    window the positions just inside it (distance window - 1) and just outside (distance window) are among them;
    the check that the plant works compares exactly these positions in the plain implementation, and that a kept
    token still carries the weight at the sequence's end."""
    folder = plant(tmp_path, dtype, kind, window, keep)
    cfg, w = RM.read_model(folder)
    n, head = 200, 120
    spots = {0, 15, 16, 17, 31, 32, 79, 81, 100, 150}
    if keep:
        spots |= {keep - 1, keep}
    for far in sorted(spots):
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
        kept = bool(window) and keep is not None and far < keep
        last_in = n - 1 if (not window or kept) else min(n - 1, far + window - 1)
        if last_in > far:                         # the key is seen up to here and carries the weight
            assert (without[last_in] - ref[last_in]).abs().max().item() > 0.5 * spread
        if window and not kept and far + window < n:           # and not one position later
            assert (without[far + window] - ref[far + window]).abs().max().item() < 1e-6 * max(1.0, spread)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, folders, oracle):
    """A short prompt, then 260 tokens one by one: the states are read and written 260 times, the pages grow
    across many borders and every window passes over decoded tokens."""
    name = "riv-a"
    toks, ref = tokens_of(name, 4), oracle(name, dtype, 4)
    r = replayer(folders, name, dtype, 320)
    outs = [r.step([dict(id="d", tokens=toks[:40], want=list(range(40)))])]
    outs += [r.step([dict(id="d", tokens=[t], want=[0])]) for t in toks[40:]]
    close(torch.cat(outs), ref, dtype, "long decoding")


# --------------------------------------------------------------------------------- kernels alone

def test_norm_kernel_that_closes_and_opens():
    from kvcm.kernels import library as K
    g = torch.Generator().manual_seed(1)
    for hidden in (40, 37, 2048):
        x = torch.randn(9, hidden, generator=g).cuda()
        y = (torch.randn(9, hidden, generator=g) * 3).cuda()
        wb, wn = (1 + 0.1 * torch.randn(hidden, generator=g)).cuda(), (1 + 0.1 * torch.randn(hidden, generator=g)).cuda()
        eps = 1e-5
        xd = x.double().cpu() + P.norm_plain(y.double().cpu(), wb.double().cpu(), eps)
        ref = P.norm_plain(xd, wn.double().cpu(), eps)
        for dtype in (torch.float32, torch.bfloat16):
            xs, out = x.clone(), torch.empty(9, hidden, dtype=dtype, device="cuda")
            K.norm_post_pre(xs, y, wb, wn, out, eps)
            assert (xs.double().cpu() - xd).abs().max().item() < 1e-5
            assert (out.double().cpu() - ref).abs().max().item() < (2e-5 if dtype == torch.float32 else 0.04)
            xs2, out2 = x.clone(), torch.empty_like(out)             # the two halves as launches of their own: the same bits
            K.norm_post_pre(xs2, y, wb, None, None, eps)
            K.norm_post_pre(xs2, None, None, wn, out2, eps)
            assert torch.equal(xs2, xs) and torch.equal(out2, out)
            rows = torch.tensor([7, 2], dtype=torch.int32, device="cuda")
            out3 = torch.empty(2, hidden, dtype=dtype, device="cuda")
            K.norm_post_pre(xs, None, None, wn, out3, eps, rows)
            assert torch.equal(out3, out[[7, 2]])


def test_polynorm_activation_kernel():
    from kvcm.kernels import library as K
    g = torch.Generator().manual_seed(2)
    for ff in (24, 333, 4096):
        z = (torch.randn(5, ff, generator=g) * 2).cuda()
        coef = torch.tensor([0.7, -0.4, 0.25, 0.1]).cuda()
        ref = P.poly_norm(z.double().cpu(), coef.double().cpu(), 1e-6)
        for dtype in (torch.float32, torch.bfloat16):
            out = torch.empty(5, ff, dtype=dtype, device="cuda")
            K.poly_norm_act(z, coef, out, 1e-6)
            assert (out.double().cpu() - ref).abs().max().item() < (2e-5 if dtype == torch.float32 else 0.05) * max(1.0, ref.abs().max().item())


def test_turning_heads_forth_and_back():
    from kvcm.kernels import library as K
    g = torch.Generator().manual_seed(3)
    T, H, HD, n = 6, 3, 24, 20
    x = torch.randn(T, H * HD, generator=g).cuda()
    pos = torch.tensor([0, 1, 7, 100, 1000, 31], dtype=torch.int32, device="cuda")
    inv = (50.0 ** (-2.0 * torch.arange(n // 2, dtype=torch.float64) / n)).float().cuda()
    for inter in (True, False):
        y = x.clone()
        K.rotate_heads(y, pos, inv, H, HD, inter, 1.0)
        xv = x.double().cpu().view(T, H, HD)
        if inter:
            ref = P.rotate_pairs(xv, pos.cpu(), 50.0, n)
        else:                                                    # halves: the same turn on a permuted vector
            perm = torch.cat([torch.arange(0, n, 2), torch.arange(1, n, 2)])
            inv_perm = torch.argsort(perm)
            t = xv.clone()
            t[..., :n] = xv[..., :n][..., inv_perm]
            t = P.rotate_pairs(t, pos.cpu(), 50.0, n)
            ref = t.clone()
            ref[..., :n] = t[..., :n][..., perm]
        assert (y.double().cpu().view(T, H, HD) - ref).abs().max().item() < 1e-4
        K.rotate_heads(y, pos, inv, H, HD, inter, -1.0)
        assert (y - x).abs().max().item() < 1e-5


def test_kept_first_keys_in_every_attention_kernel():
    """The tensor-core attention kernels (decode in one block, split over a cluster, split through scratch
    memory; prefill) against the plain kernel, with a window, kept first tokens and a sink; contexts in which the
    kept keys share a tile with the window, lie tiles before it, and outnumber a tile."""
    for window, keep, hd in ((100, 7, 64), (300, 70, 96), (64, 130, 32), (500, 1, 128), (200, 130, 64), (129, 64, 128)):
        layer = {"type": "attention", "mixer": RM.attn(8, 2, hd, hd - 16, 0.2, (10000.0, 16), window, keep), "mlp": None}
        import tempfile
        folder = RM.write_model_from({"architecture": "Rivetar", "vocab": 64, "width": 64, "norm": {"eps": 1e-6},
                                      "layers": [layer]}, 3, "bfloat16", tempfile.mkdtemp())
        toks = helpers.random_tokens(900, 64, 8)
        outs = {}
        for options in ({"attention": "plain"}, {"attn_parts": 1}, {"attn_parts": 4}, {"attn_parts": 4, "attn_merge": "kernel"},
                        {"attn_prefill": "mma"}, {}):
            r = helpers.Replayer(folder, "bfloat16", 1024, 16, options=options)
            o = [r.step([dict(id="a", tokens=toks[:50], want=[3, 49])]),
                 r.step([dict(id="a", tokens=toks[50:880], want=list(range(0, 830, 23)) + [829])])]
            o += [r.step([dict(id="a", tokens=[t], want=[0])]) for t in toks[880:]]
            outs[json.dumps(options)] = torch.cat(o)
        base = outs.pop(json.dumps({"attention": "plain"}))
        for name, o in outs.items():
            close(o, base, "bfloat16", f"window {window} keep {keep}: {name}")


def test_latent_attention_prefill_kernels_agree():
    """Attention over a cached latent whose page row has 256 elements (keys and values are the same pages): the
    default prefill kernel against the plain kernel and the other tensor-core one, in portions cut at odd places,
    beside a second request."""
    import tempfile
    layer = {"type": "latent_attention", "mixer": RM.latent(6, 96, 64, 80, 192, 128, 0.06, (10000.0, 64)), "mlp": None}
    folder = RM.write_model_from({"architecture": "Rivetar", "vocab": 64, "width": 128, "norm": {"eps": 1e-6},
                                  "layers": [layer]}, 5, "bfloat16", tempfile.mkdtemp())
    toks, other = helpers.random_tokens(700, 64, 9), helpers.random_tokens(333, 64, 10)
    outs = {}
    for options in ({"attention": "plain"}, {"attn_prefill": "mma"}, {}):
        r = helpers.Replayer(folder, "bfloat16", 1152, 16, options=options)
        o = [r.step([dict(id="a", tokens=toks[:131], want=[0, 1, 63, 64, 130])]),
             r.step([dict(id="a", tokens=toks[131:690], want=list(range(0, 559, 29)) + [558]),
                     dict(id="b", tokens=other, want=[0, 127, 128, 332])])]
        o += [r.step([dict(id="a", tokens=[t], want=[0])]) for t in toks[690:]]
        outs[json.dumps(options)] = torch.cat(o)
    base = outs.pop(json.dumps({"attention": "plain"}))
    for name, o in outs.items():
        close(o, base, "bfloat16", f"latent rows of 256: {name}")


def test_blocks_with_and_without_the_fused_norms(folders, oracle):
    """The norm that closes the mixer and the norm that opens the feed-forward as one launch or as two: the same
    logits bit for bit."""
    name, dtype = "riv-a", "bfloat16"
    toks = tokens_of(name, 3)
    outs = []
    for options in ({}, {"fuse": False}):
        r = replayer(folders, name, dtype, 320, options=options)
        outs.append(r.step([dict(id="a", tokens=toks, want=list(range(len(toks))))], end=["a"]))
    assert torch.equal(outs[0], outs[1])


# -------------------------------------------------------------- the engine's own entry point

@pytest.mark.parametrize("name", ["riv-a", "riv-c"])
def test_greedy_generation_through_the_engine(name, folders):
    """Scheduler with chunked prefill and few sequences at a time; every generated token must be the plain
    implementation's choice given the tokens before it (ties within 2e-4 allowed)."""
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    folder = folders(name, "float32")
    cfg, w = RM.read_model(folder)
    B = RM.CONFIGS[name]["block_size"]
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
    assert eng.kv.blocks_in_use(0) == 0 and eng.sched.slots_taken() == 0
    eng2, outs2 = run(False)
    assert eng2.graphs is None and outs2 == outs


def test_generation_in_bfloat16_with_eviction(folders):
    """So few pages that running requests are evicted and computed again from their first token: the state slot
    is reset.  With room for all and without, every generated token is the plain implementation's choice given
    the tokens before it, or within the bfloat16 engine's rounding of it (recomputing a request as one portion
    rounds differently from decoding it token by token, so near-ties may fall the other way)."""
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    folder = folders("riv-a", "bfloat16")
    cfg, w = RM.read_model(folder)
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
    assert [o[:8] for o in outs2] == [o[:8] for o in outs]


def test_trace_tool_on_a_model_folder(tmp_path, folders, oracle):
    name, dtype = "riv-b", "float32"
    toks, ref = tokens_of(name, 2), oracle(name, dtype, 2)
    other = tokens_of(name, 1)
    steps = [dict(step=0, entries=[dict(id="a", tokens=toks[:70], want=[0, 69])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=toks[70:72], want=[1]), dict(id="b", tokens=other, want=[63])], end=["b"]),
             dict(step=2, entries=[dict(id="a", tokens=toks[72:], want=[len(toks) - 73])], end=["a"])]
    out = helpers.run_trace_tool(folders(name, dtype), dtype, steps, 512, str(tmp_path / "out"), vocab_key="vocab")
    got = torch.cat([torch.from_numpy(out[0]), torch.from_numpy(out[1][:1]), torch.from_numpy(out[2])])
    close(got, ref[[0, 69, 71, len(toks) - 1]], dtype, "trace tool")
    close(torch.from_numpy(out[1][1:]), oracle(name, dtype, 1)[[63]], dtype, "trace tool, second request")
