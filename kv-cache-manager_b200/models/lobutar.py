"""Lobutar assembled from parts (registered as ``Lobutar``).

The residual stream is ``streams`` copies of the embedding's output (hyper-connections: every sublayer reads a learned
sum of the streams through an RMS norm and writes its output back through a learned mix; the model's output is the sum
of the streams).  Every layer is a "hyper_connection" block whose mixer is, by the layer's ``type``,

* "attention": differential attention, two softmax maps per head over the same values, subtracted, normalised per head
  and gated per head (``differential_attention``), biased projections, partial rotary encoding in interleaved pairs;
* "latent_attention": attention over a cached latent with a shared rotated key part, queries straight from the
  input, a sliding window, a sink per head and an element-wise output gate (``latent_rope_attention``);

and whose feed-forward is absent, dense (SiLU-gated) or a set of routed experts (sigmoid scores, a correction for the
choice only, groups scored by their two largest choice scores, weights not renormalised) with an ungated shared
expert.  A layer with ``weights_of: j`` is a second run-order entry of layer j's block: same parts and tensors, pages
of its own.  Final norm over the sum of the streams, output head.

Checkpoint names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.hc1|hc2.in|out|mix``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``; linear weights [out, in].  Fused at load: q|k|v|g of an attention mixer (and its three
biases), q|dkv|g of a latent mixer, gate|up of a dense or shared feed-forward, the experts' matrices stacked.
"""
from __future__ import annotations

from ..config.model_config import LobutarConfig
from ..config.registry import register_architecture
from ..parts.base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, LayerCall
from ..parts.embedding import LMHead
from ..parts.hyper import StreamsEmbedding
from .spec import ModelSpec, TensorBinding


def _gated(bindings, ffn, prefix: str, D: int, F: int) -> None:
    bindings += [TensorBinding(ffn.gate_up, "weight", [(prefix + "gate", (F, D)), (prefix + "up", (F, D))]),
                 TensorBinding(ffn.down, "weight", [(prefix + "down", (D, F))])]


def build_lobutar(cfg: LobutarConfig, norm_init=("ones_jitter", 0.1)) -> ModelSpec:
    D, eps, S = cfg.width, cfg.norm_eps, cfg.streams
    embedding = StreamsEmbedding(cfg.vocab, D, S)
    bindings = [TensorBinding(embedding, "weight", [("embed", (cfg.vocab, D))])]
    blocks, order, block_of, ignorable = [], [], {}, []
    for i, layer in enumerate(cfg.layers):
        if layer.get("weights_of") is not None:          # another run of an earlier layer's block, with pages of its own
            block_of[i] = block_of[int(layer["weights_of"])]
            order.append(LayerCall(block_of[i]))
            continue
        m, p = layer["mixer"], f"l{i}.mix."
        rot = m.get("rot")
        if layer["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            position = (POSITION_ENCODINGS.build("rope", head_dim=dk, theta=rot["base"], rotary_dim=rot["dims"], pairing="interleaved")
                        if rot else POSITION_ENCODINGS.build("none"))
            mixer = MIXERS.build("differential_attention", hidden=D, num_heads=H, num_kv_heads=G, dk=dk, dv=dv,
                                 position=position, diff=m["diff"], scale=m["scale"], norm_eps=eps)
            bindings += [TensorBinding(mixer.qkvg, "weight", [(p + "q", (H * 2 * dk, D)), (p + "k", (G * 2 * dk, D)),
                                                              (p + "v", (G * dv, D)), (p + "g", (H, D))]),
                         TensorBinding(mixer, "bias", [(p + "q.b", (H * 2 * dk,)), (p + "k.b", (G * 2 * dk,)), (p + "v.b", (G * dv,))]),
                         TensorBinding(mixer.o, "weight", [(p + "o", (D, H * dv))]),
                         TensorBinding(mixer, "o_bias", [(p + "o.b", (D,))])]
            bindings += [TensorBinding(mixer, n, [(p + n, (dk,))]) for n in ("lq1", "lk1", "lq2", "lk2")]
        else:                                             # "latent_attention" (the config has been validated)
            H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            position = POSITION_ENCODINGS.build("rope", head_dim=dr, theta=rot["base"], rotary_dim=rot["dims"], pairing="interleaved")
            mixer = MIXERS.build("latent_rope_attention", hidden=D, heads=H, dn=dn, dr=dr, dv=dv, rank=R, q_rank=0,
                                 scale=m["scale"], norm_eps=eps, position=position, window=(m.get("mask") or {}).get("size", 0),
                                 sink=True, gate=True)
            bindings += [TensorBinding(mixer.dq_dkv, "weight", [(p + "q", (H * (dn + dr), D)), (p + "dkv", (R + dr, D)),
                                                                (p + "g", (H * dv, D))]),
                         TensorBinding(mixer, "latent_norm", [(p + "dkv.norm", (R,))]),
                         TensorBinding(mixer.uk, "weight", [(p + "uk", (H * dn, R))]),
                         TensorBinding(mixer.uv, "weight", [(p + "uv", (H * dv, R))]),
                         TensorBinding(mixer, "sink", [(p + "sink", (H,))]),
                         TensorBinding(mixer.o, "weight", [(p + "o", (D, H * dv))])]
        norm1 = NORMS.build("rmsnorm", hidden=D, eps=eps, init=norm_init)
        bindings.append(TensorBinding(norm1, "weight", [(f"l{i}.norm1", (D,))]))
        norm2 = ffn = None
        mlp = layer.get("mlp")
        if mlp is None:                                   # a checkpoint may still carry the unused second sublayer's small tensors
            ignorable += [f"l{i}.norm2", f"l{i}.hc2."]
        if mlp is not None:
            q = f"l{i}.mlp."
            if mlp["kind"] == "dense":
                ffn = FEED_FORWARDS.build("gated_mlp", hidden=D, intermediate=mlp["ff"])
                _gated(bindings, ffn, q, D, mlp["ff"])
            else:
                r = mlp["router"]
                E, F = r["experts"], mlp["expert"]["ff"]
                groups = r.get("groups") or {"count": 1, "keep": 1}
                shared_ff = (mlp.get("shared") or {}).get("ff", 0)
                ffn = FEED_FORWARDS.build("routed_experts", hidden=D, experts=E, expert_ff=F, top=r["top"], scale=r.get("scale", 1.0),
                                          groups=groups["count"], keep=groups["keep"], shared_ff=shared_ff, scores="sigmoid",
                                          correction=True, group_top=2, shared_gate=False)
                bindings += [TensorBinding(ffn, "router", [(q + "router", (E, D))]),
                             TensorBinding(ffn, "correction", [(q + "correction", (E,))]),
                             TensorBinding(ffn, "gate_up", [(f"{q}e{e}.{n}", (F, D)) for e in range(E) for n in ("gate", "up")]),
                             TensorBinding(ffn, "down", [(f"{q}e{e}.down", (D, F)) for e in range(E)])]
                if shared_ff:
                    _gated(bindings, ffn.shared, q + "shared.", D, shared_ff)
            norm2 = NORMS.build("rmsnorm", hidden=D, eps=eps, init=norm_init)
            bindings.append(TensorBinding(norm2, "weight", [(f"l{i}.norm2", (D,))]))
        block = BLOCKS.build("hyper_connection", streams=S, norm1=norm1, mixer=mixer, norm2=norm2, ffn=ffn)
        for hc, name in ((block.hc1, "hc1"), (block.hc2, "hc2")):
            if hc is not None:
                bindings += [TensorBinding(hc, "in", [(f"l{i}.{name}.in", (S,))]),
                             TensorBinding(hc, "out", [(f"l{i}.{name}.out", (S,))]),
                             TensorBinding(hc, "mix", [(f"l{i}.{name}.mix", (S, S))])]
        block_of[i] = len(blocks)
        blocks.append(block)
        order.append(LayerCall(block_of[i]))
    final_norm = NORMS.build("rmsnorm_streams", hidden=D, eps=eps, streams=S, init=norm_init)
    bindings.append(TensorBinding(final_norm, "weight", [("final.norm", (D,))]))
    head = LMHead(D, cfg.vocab)
    bindings.append(TensorBinding(head, "weight", [("head", (cfg.vocab, D))]))
    return ModelSpec(cfg, embedding, blocks, order, final_norm, head, bindings, ignorable=tuple(ignorable))


register_architecture("Lobutar", LobutarConfig, build_lobutar, replace=True)
