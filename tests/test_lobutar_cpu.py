"""Lobutar without a GPU: the configuration reader and its refusals, the builder's tensor names, shapes and run
order, and the plain implementation's own pieces against closed forms."""
import copy
import json
import math

import pytest
import torch

import lobutar_models as LM
import plain_lobutar as P


def test_config_is_read_and_written_back():
    import kvcm
    for name, c in LM.CONFIGS.items():
        cfg = kvcm.config.config_from_dict(c["cfg"])
        assert cfg.architecture == "Lobutar" and cfg.width == c["cfg"]["width"] and cfg.streams == c["cfg"]["streams"]
        assert kvcm.config.config_from_dict(cfg.to_json_dict()) == cfg


@pytest.mark.parametrize("edit,word", [
    (lambda d: d["layers"][0].__setitem__("type", "conv"), "unknown type"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 14), "within"),
    (lambda d: d["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda d: d["layers"][1]["mixer"]["rot"].__setitem__("dims", 10), "rot_dim"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][1]["mixer"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda d: d["layers"][1]["mlp"]["router"].__setitem__("top", 5), "choices"),
    (lambda d: d["layers"][1]["mlp"]["router"]["groups"].__setitem__("count", 3), "choices"),
    (lambda d: d["layers"][1]["mlp"].pop("expert"), "expert"),
    (lambda d: d["layers"][0].__setitem__("mlp", {"kind": "conv"}), "dense"),
    (lambda d: d["layers"][2].__setitem__("weights_of", 2), "weights_of"),
    (lambda d: d["layers"][4].__setitem__("weights_of", 7), "weights_of"),
    (lambda d: d["layers"][4].__setitem__("weights_of", 0), "same type"),
    (lambda d: d.__setitem__("streams", 0), "streams"),
    (lambda d: d.pop("norm"), "norm"),
])
def test_config_refusals_name_the_key(edit, word):
    import kvcm
    d = json.loads(json.dumps(LM.CONFIGS["lob-a"]["cfg"]))          # (layers that share weights share no objects)
    edit(d)
    with pytest.raises(kvcm.config.ConfigError) as e:
        kvcm.config.config_from_dict(d)
    assert word in str(e.value)


def test_builder_names_every_tensor_once_and_runs_shared_layers_twice():
    import kvcm
    from kvcm.engine.model_io import build_spec
    from kvcm.cache.pools import plan_cache
    cfg = kvcm.config.config_from_dict(copy.deepcopy(LM.CONFIGS["lob-a"]["cfg"]))
    spec = build_spec(cfg)
    names = [n for b in spec.bindings for n, _ in b.sources]
    assert len(names) == len(set(names))
    for want in ("embed", "l0.norm1", "l0.norm2", "l0.hc1.in", "l0.hc2.mix", "l0.mix.q.b", "l0.mix.o.b", "l0.mix.lk2", "l0.mix.g",
                 "l0.mlp.gate", "l1.mix.dkv.norm", "l1.mix.sink", "l1.mix.g", "l1.mlp.router", "l1.mlp.correction", "l1.mlp.e7.down",
                 "l1.mlp.shared.up", "l3.mix.uk", "l3.hc1.out", "final.norm", "head"):
        assert want in names, want
    assert not any(n.startswith(("l2.", "l4.")) for n in names)           # layers that run with another layer's weights
    assert "l3.norm2" not in names and "l3.hc2.in" not in names
    shapes = dict(s for b in spec.bindings for s in b.sources)
    assert shapes["l0.mix.q"] == (4 * 2 * 12, 72) and shapes["l0.mix.k"] == (2 * 2 * 12, 72) and shapes["l0.mix.g"] == (4, 72)
    assert shapes["l1.mix.dkv"] == (40 + 8, 72) and shapes["l1.mix.g"] == (3 * 20, 72) and shapes["l0.hc1.mix"] == (3, 3)
    assert [c.layer for c in spec.order] == [0, 1, 0, 2, 1] and len(spec.blocks) == 3
    plan = plan_cache(spec)
    assert all(plan.site_writes) and len({(g, l) for g, l in zip(plan.site_group, plan.site_layer)}) == 5   # pages of its own per run
    windows = sorted(plan.windows)
    assert windows == [0, 0, 37]


def test_a_layer_may_name_a_layer_that_itself_borrows_its_weights():
    import kvcm
    from kvcm.engine.model_io import build_spec
    d = json.loads(json.dumps(LM.CONFIGS["lob-a"]["cfg"]))
    d["layers"].append(dict(d["layers"][2], weights_of=2))                # layer 5 -> layer 2 -> layer 0
    spec = build_spec(kvcm.config.config_from_dict(d))
    assert [c.layer for c in spec.order] == [0, 1, 0, 2, 1, 0] and len(spec.blocks) == 3


def test_plain_rotation_and_visibility():
    x = torch.arange(24, dtype=P.F).view(2, 1, 12) + 1.0
    pos = torch.tensor([0, 5])
    y = P.rotate_pairs(x, pos, 100.0, 4)
    assert torch.equal(y[0], x[0]) and torch.equal(y[1, :, 4:], x[1, :, 4:])
    a = 5 * 100.0 ** (-2.0 / 4)
    assert y[1, 0, 2].item() == pytest.approx(x[1, 0, 2].item() * math.cos(a) - x[1, 0, 3].item() * math.sin(a))
    assert y[1, 0, 1].item() == pytest.approx(x[1, 0, 1].item() * math.cos(5.0) + x[1, 0, 0].item() * math.sin(5.0))
    v = P.visible(6, 3)
    assert v[5].tolist() == [False, False, False, True, True, True] and v[1].tolist() == [True, True, False, False, False, False]
    assert P.visible(4).tolist() == torch.tril(torch.ones(4, 4)).bool().tolist()


def test_plain_softmax_sink_counts_once_and_has_no_value():
    s = torch.zeros(1, 2, 2, dtype=P.F)
    p = P.softmax_visible(s, P.visible(2), torch.tensor([math.log(2.0)], dtype=P.F))
    assert p[0, 0].tolist() == pytest.approx([1 / 3, 0.0]) and p[0, 1].tolist() == pytest.approx([0.25, 0.25])


def test_plain_streams_and_router():
    xs = torch.tensor([[[1.0, 2.0]], [[10.0, 20.0]]], dtype=P.F)                 # two streams, one token, width 2
    hc = {"in": torch.tensor([2.0, 0.5], dtype=P.F), "out": torch.tensor([1.0, -1.0], dtype=P.F),
          "mix": torch.tensor([[1.0, 3.0], [0.0, 2.0]], dtype=P.F)}               # [from, to]
    assert P.hyper_read(xs, hc).tolist() == [[7.0, 14.0]]
    new = P.hyper_write(xs, torch.tensor([[100.0, 200.0]], dtype=P.F), hc)
    assert new[0].tolist() == [[101.0, 202.0]] and new[1].tolist() == [[3 + 20 - 100.0, 6 + 40 - 200.0]]
    # four experts in two groups, one kept: the group with the larger sum of its two choice scores wins although
    # the single best expert lies in the other one; the correction counts for the choice, not for the weight
    w = {"router": torch.eye(4, dtype=P.F), "correction": torch.tensor([0.0, 0.0, 0.3, 0.3], dtype=P.F)}
    h = torch.tensor([[3.0, -3.0, 1.0, 1.0]], dtype=P.F)
    idx, wt = P.route(h, w, {"experts": 4, "top": 1, "groups": {"count": 2, "keep": 1}, "scale": 2.0})
    assert idx.tolist() in ([[2]], [[3]]) and wt.item() == pytest.approx(2.0 / (1.0 + math.exp(-1.0)))
    w["correction"] = torch.tensor([-5.0, -5.0, -6.0, -7.0], dtype=P.F)           # all choice scores negative
    idx, wt = P.route(h, w, {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}})
    assert sorted(idx[0].tolist()) == [0, 1]


def test_plain_differential_lambda_and_whole_model_runs():
    w = {n: torch.full((3,), v, dtype=P.F) for n, v in (("lq1", 0.1), ("lk1", 1.0), ("lq2", 0.2), ("lk2", 0.5))}
    assert P.differential_lambda(w, 0.25).item() == pytest.approx(math.exp(0.3) - math.exp(0.3) + 0.25)
    import kvcm
    c = LM.CONFIGS["lob-c"]
    cfg = kvcm.config.config_from_dict(c["cfg"])
    tensors = {n: t.double() for n, t in kvcm.weights.random_init.random_tensors(cfg, 3, torch.float32)}
    logits, after = P.trace(c["cfg"], tensors, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 97) and len(after) == 3 and torch.isfinite(logits).all()
    again = P.forward(c["cfg"], tensors, [1, 2, 3])
    assert torch.allclose(again, logits[:3], atol=1e-12)                         # causal: a prefix gives the same rows
