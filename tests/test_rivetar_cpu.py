"""Rivetar without a GPU: the configuration reader and its refusals, the builder's tensor names, shapes and run
order, and the plain implementation's own pieces against each other."""
import copy

import pytest
import torch

import plain_rivetar as P
import rivetar_models as RM


def test_config_is_read_and_written_back():
    import kvcm
    for name, c in RM.CONFIGS.items():
        cfg = kvcm.config.config_from_dict(c["cfg"])
        assert cfg.architecture == "Rivetar" and cfg.width == c["cfg"]["width"]
        assert kvcm.config.config_from_dict(cfg.to_json_dict()) == cfg
    d = copy.deepcopy(RM.CONFIGS["riv-b"]["cfg"])
    d.pop("embedding")
    cfg = kvcm.config.config_from_dict(d)
    assert cfg.embedding_scale == 1.0 and cfg.logit_softcap == 0.0 and not cfg.has_loop


@pytest.mark.parametrize("edit,word", [
    (lambda d: d["layers"][0].__setitem__("type", "conv"), "unknown type"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 26), "within"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("vdim", 41), "vdim"),
    (lambda d: d["layers"][0]["mixer"]["mask"].__setitem__("keep_first", -1), "keep_first"),
    (lambda d: d["layers"][1]["mixer"].__setitem__("tau", 0.0), "tau"),
    (lambda d: d["layers"][2]["mixer"]["rot"].__setitem__("dims", 10), "rot_dim"),
    (lambda d: d["layers"][2]["mixer"].pop("q_rank"), "q_rank"),
    (lambda d: d["loop"].__setitem__("stop", 9), "loop"),
    (lambda d: d["loop"].__setitem__("times", 0), "loop"),
    (lambda d: d["layers"][0].__setitem__("mlp", {"kind": "moe"}), "dense"),
    (lambda d: d.pop("norm"), "norm"),
])
def test_config_refusals_name_the_key(edit, word):
    import kvcm
    d = copy.deepcopy(RM.CONFIGS["riv-a"]["cfg"])
    edit(d)
    with pytest.raises(kvcm.config.ConfigError) as e:
        kvcm.config.config_from_dict(d)
    assert word in str(e.value)


def test_builder_names_every_tensor_once_and_takes_the_decay_rank_from_shapes():
    import kvcm
    from kvcm.engine.model_io import build_spec
    d = copy.deepcopy(RM.CONFIGS["riv-a"]["cfg"])
    cfg = kvcm.config.config_from_dict(d)
    spec = build_spec(cfg)
    names = [n for b in spec.bindings for n, _ in b.sources]
    assert len(names) == len(set(names))
    for want in ("embed", "loop.in", "loop.step", "l0.norm1b", "l0.norm2b", "l0.mix.sink", "l0.mlp.act", "l1.mix.a2.b",
                 "l1.mix.norm", "l2.mix.dq.norm", "l2.mix.dkv.norm", "l2.mix.uk", "l4.mix.uv", "final.norm", "head"):
        assert want in names, want
    assert "l1.norm2" not in names and "l1.mlp.up" not in names and "l3.norm2b" not in names
    shapes = dict(s for b in spec.bindings for s in b.sources)
    assert shapes["l1.mix.a1"] == (5, 72) and shapes["l1.mix.a2"] == (60, 5) and shapes["loop.step"] == (3, 72)
    assert shapes["l2.mix.dkv"] == (48, 72) and shapes["l2.mix.uq"] == (72, 24) and shapes["loop.in"] == (72, 144)
    d["layers"][1]["mixer"].pop("decay_rank")
    cfg2 = kvcm.config.config_from_dict(d)
    with pytest.raises(kvcm.config.ConfigError):
        build_spec(cfg2)
    spec2 = build_spec(cfg2, {"l1.mix.a1": (7, 72)})
    assert dict(s for b in spec2.bindings for s in b.sources)["l1.mix.a2"] == (60, 7)


def test_run_order_of_a_looped_span():
    """Every pass is a run-order entry of its own (own pages and state rows); the first layer of each pass is
    entered through the loop's part with the number of the pass."""
    import kvcm
    from kvcm.cache.pools import plan_cache
    from kvcm.engine.model_io import build_spec
    spec = build_spec(kvcm.config.config_from_dict(RM.CONFIGS["riv-a"]["cfg"]))
    assert [c.layer for c in spec.order] == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert [c.enter[1] if c.enter else None for c in spec.order] == [None, 0, None, 1, None, 2, None, None, None]
    assert [(i, t) for i, t, _ in P.run_order(RM.CONFIGS["riv-a"]["cfg"])] == \
        [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (1, 2), (2, 2), (3, None), (4, None)]
    plan = plan_cache(spec)
    assert sum(s is not None for s in plan.site_state) == 3                     # the gla layer, once per pass
    assert all(g.spec.window == 0 for g in plan.groups if g.spec.num_kv_heads == 2)   # kept first tokens: pages stay
    spec_b = build_spec(kvcm.config.config_from_dict(RM.CONFIGS["riv-b"]["cfg"]))
    assert [c.layer for c in spec_b.order] == [0, 1, 2, 3] and not spec_b.extras
    windows = sorted(g.spec.window for g in plan_cache(spec_b).groups)
    assert windows == [0, 0, 70]                    # a plain window gives pages back; one with kept tokens does not


def test_plain_pieces_agree_with_each_other():
    g = torch.Generator().manual_seed(4)
    x = torch.randn(7, 3, 12, generator=g, dtype=torch.float64)
    pos = torch.tensor([0, 1, 5, 40, 41, 1000, 77])
    y = P.rotate_pairs(x, pos, 300.0, 8)
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.equal(y[0], x[0])
    assert (P.rotate_pairs(y, pos, 300.0, 8, sign=-1.0) - x).abs().max().item() < 1e-12
    # a turn keeps every pair's length, and the product of two turned vectors depends on the distance only
    assert ((y[..., 0:8:2] ** 2 + y[..., 1:8:2] ** 2) - (x[..., 0:8:2] ** 2 + x[..., 1:8:2] ** 2)).abs().max().item() < 1e-12
    a, b = torch.randn(1, 1, 8, generator=g, dtype=torch.float64), torch.randn(1, 1, 8, generator=g, dtype=torch.float64)
    d1 = (P.rotate_pairs(a, torch.tensor([9]), 50.0, 8) * P.rotate_pairs(b, torch.tensor([4]), 50.0, 8)).sum()
    d2 = (P.rotate_pairs(a, torch.tensor([105]), 50.0, 8) * P.rotate_pairs(b, torch.tensor([100]), 50.0, 8)).sum()
    assert abs(d1.item() - d2.item()) < 1e-9
    m = P.visible(12, 4, 2)
    assert m[11].tolist() == [True, True] + [False] * 6 + [True] * 4 and m[3].tolist() == [True] * 4 + [False] * 8
    assert torch.equal(P.visible(6), torch.tril(torch.ones(6, 6, dtype=torch.bool)))
    s = torch.randn(2, 5, 5, generator=g, dtype=torch.float64)
    p = P.softmax_with_sink(s, P.visible(5), torch.tensor([0.3, -2.0], dtype=torch.float64))
    total = p.sum(-1)
    assert (total < 1).all() and (p.masked_select(~P.visible(5)[None].expand(2, 5, 5)) == 0).all()
    e = torch.exp(torch.tensor(0.3, dtype=torch.float64))
    want = 1 - e / (torch.exp(s[0, 0, 0]) + e)
    assert abs(total[0, 0].item() - want.item()) < 1e-12
    z = torch.randn(3, 16, generator=g, dtype=torch.float64)
    out = P.poly_norm(z, torch.tensor([0.0, 1.0, 0.0, 0.5]), 0.0)
    assert ((out - 0.5) ** 2).mean(-1).sub(1).abs().max().item() < 1e-12          # N(z^2) has unit mean square


def test_plain_gla_state_against_its_closed_form():
    """o_t = sum_{s<=t} (q_t . (prod_{s<r<=t} alpha_r) k_s) v_s."""
    g = torch.Generator().manual_seed(5)
    T, D, H, dk, dv, r = 9, 16, 2, 4, 6, 3
    m = {"heads": H, "dim": dk, "vdim": dv, "tau": 3.0}
    w = {n: torch.randn(*s, generator=g, dtype=torch.float64) * 0.5 for n, s in
         dict(q=(H * dk, D), k=(H * dk, D), v=(H * dv, D), g=(H * dv, D), o=(D, H * dv), a1=(r, D), a2=(H * dk, r)).items()}
    w["a2.b"] = torch.randn(H * dk, generator=g, dtype=torch.float64)
    w["norm"] = torch.ones(dv, dtype=torch.float64)
    h = torch.randn(T, D, generator=g, dtype=torch.float64)
    got = P.mixer_gla(h, m, w, 1e-6)
    q = (h @ w["q"].T).view(T, H, dk) * dk ** -0.5
    k, v = (h @ w["k"].T).view(T, H, dk), (h @ w["v"].T).view(T, H, dv)
    la = torch.log(torch.sigmoid((h @ w["a1"].T) @ w["a2"].T + w["a2.b"])).view(T, H, dk) / 3.0
    o = torch.zeros(T, H, dv, dtype=torch.float64)
    for t in range(T):
        for s in range(t + 1):
            decay = torch.exp(la[s + 1:t + 1].sum(0))
            o[t] += ((q[t] * decay * k[s]).sum(-1, keepdim=True)) * v[s]
    gate = h @ w["g"].T
    want = (P.norm_plain(o, w["norm"], 1e-6).reshape(T, H * dv) * gate * torch.sigmoid(gate)) @ w["o"].T
    assert (got - want).abs().max().item() < 1e-10
