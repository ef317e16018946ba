"""Rivetar assembled from parts (registered as ``Rivetar``).

Embedding times a constant; every layer is a "sandwich" block, x += norm_b(sublayer(norm(x))) for the mixer and,
where the layer has one, for the feed-forward, all norms RMS norms whose weights are stored around zero; the
mixer is, by the layer's ``type``,

* "latent_attention": attention over a cached latent with a shared rotated key part and queries through a
  latent of their own (``latent_rope_attention``);
* "attention": grouped-query attention with partial rotary encoding in interleaved pairs, values that are
  turned by their position and turned back at the reader, a sliding window that keeps a request's first
  tokens, and a sink per head (``attention_general``);
* "gla": gated linear attention with a decay per key channel (``gla``);

the feed-forward is absent or dense with the PolyNorm activation.  A span of layers may run several times in a
row with the same weights: every pass is a run-order entry of its own (own pages, own state), and the first
layer of each pass is entered through ``LoopEntry``, which mixes the stream with the embedding's output and adds
the pass's row.  Final norm, output head, logits capped by a tanh.

Checkpoint names: ``embed``, ``loop.in``, ``loop.step``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``,
``l<i>.mlp.up|down|act``, ``final.norm``, ``head``; linear weights [out, in].  Fused at load: dq|dkv of a latent
mixer, q|k|v of the other two.  The rank of a gla mixer's two-stage decay projection is the shape of its tensor
(``tensor_shapes``, from the checkpoint's header) or, when a model is made without a checkpoint, the optional
mixer key ``decay_rank``.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

from ..config.model_config import ConfigError, RivetarConfig
from ..config.registry import register_architecture
from ..parts.base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, LayerCall
from ..parts.embedding import LMHead, ScaledEmbedding
from ..parts.loop import LoopEntry
from .spec import ModelSpec, TensorBinding


def _norm(bindings, name: str, D: int, eps: float, init):
    norm = NORMS.build("rmsnorm_offset", hidden=D, eps=eps, init=init)
    bindings.append(TensorBinding(norm, "weight", [(name, (D,))]))
    return norm


def build_rivetar(cfg: RivetarConfig, norm_init=("normal", 0.1),
                  tensor_shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> ModelSpec:
    D, eps = cfg.width, cfg.norm_eps
    keep = "x0" if cfg.has_loop else None
    embedding = ScaledEmbedding(cfg.vocab, D, scale=cfg.embedding_scale, keep_as=keep)
    bindings = [TensorBinding(embedding, "weight", [("embed", (cfg.vocab, D))])]
    blocks = []
    for i, layer in enumerate(cfg.layers):
        m, p, kind = layer["mixer"], f"l{i}.mix.", layer["type"]
        if kind == "latent_attention":
            H, dn, dr, dv, R, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            position = POSITION_ENCODINGS.build("rope", head_dim=dr, theta=m["rot"]["base"], rotary_dim=m["rot"]["dims"],
                                                pairing="interleaved")
            mixer = MIXERS.build("latent_rope_attention", hidden=D, heads=H, dn=dn, dr=dr, dv=dv, rank=R, q_rank=qr,
                                 scale=m["scale"], norm_eps=eps, position=position)
            bindings += [TensorBinding(mixer.dq_dkv, "weight", [(p + "dq", (qr, D)), (p + "dkv", (R + dr, D))]),
                         TensorBinding(mixer, "q_norm", [(p + "dq.norm", (qr,))]),
                         TensorBinding(mixer, "latent_norm", [(p + "dkv.norm", (R,))]),
                         TensorBinding(mixer.uq, "weight", [(p + "uq", (H * (dn + dr), qr))]),
                         TensorBinding(mixer.uk, "weight", [(p + "uk", (H * dn, R))]),
                         TensorBinding(mixer.uv, "weight", [(p + "uv", (H * dv, R))]),
                         TensorBinding(mixer.o, "weight", [(p + "o", (D, H * dv))])]
        elif kind == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            mask = m.get("mask") or {}
            position = POSITION_ENCODINGS.build("rope", head_dim=dk, theta=m["rot"]["base"], rotary_dim=m["rot"]["dims"],
                                                pairing="interleaved")
            mixer = MIXERS.build("attention_general", hidden=D, num_heads=H, num_kv_heads=G, dk=dk, dv=dv, position=position,
                                 scale=m["scale"], window=mask.get("size", 0), keep_first=mask.get("keep_first", 0) or 0,
                                 sink=True, norm_eps=eps, rotate_values=True)
            bindings += [TensorBinding(mixer.qkv, "weight", [(p + "q", (H * dk, D)), (p + "k", (G * dk, D)), (p + "v", (G * dv, D))]),
                         TensorBinding(mixer.o, "weight", [(p + "o", (D, H * dv))]),
                         TensorBinding(mixer, "sink", [(p + "sink", (H,))])]
        else:                                       # "gla" (the config has been validated)
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            name = p + "a1"
            if tensor_shapes is not None and name in tensor_shapes and len(tensor_shapes[name]) == 2:
                ra = int(tensor_shapes[name][0])
            elif isinstance(m.get("decay_rank"), int) and m["decay_rank"] > 0:
                ra = m["decay_rank"]
            else:
                raise ConfigError(f"Rivetar: the rank of '{name}' is given neither by a tensor's shape nor by mixer key 'decay_rank'")
            mixer = MIXERS.build("gla", hidden=D, heads=H, dk=dk, dv=dv, decay_rank=ra, tau=m["tau"], norm_eps=eps)
            bindings += [TensorBinding(mixer.qkv, "weight", [(p + "q", (H * dk, D)), (p + "k", (H * dk, D)), (p + "v", (H * dv, D))]),
                         TensorBinding(mixer.g, "weight", [(p + "g", (H * dv, D))]),
                         TensorBinding(mixer.a1, "weight", [(p + "a1", (ra, D))]),
                         TensorBinding(mixer.a2, "weight", [(p + "a2", (H * dk, ra))]),
                         TensorBinding(mixer, "a2_bias", [(p + "a2.b", (H * dk,))]),
                         TensorBinding(mixer, "norm", [(p + "norm", (dv,))]),
                         TensorBinding(mixer.o, "weight", [(p + "o", (D, H * dv))])]
        norm1 = _norm(bindings, f"l{i}.norm1", D, eps, norm_init)
        norm1b = _norm(bindings, f"l{i}.norm1b", D, eps, norm_init)
        norm2 = ffn = norm2b = None
        mlp = layer.get("mlp")
        if mlp is not None:
            ffn = FEED_FORWARDS.build("dense_mlp", hidden=D, intermediate=mlp["ff"], activation="polynorm", norm_eps=eps)
            bindings += [TensorBinding(ffn.up, "weight", [(f"l{i}.mlp.up", (mlp["ff"], D))]),
                         TensorBinding(ffn.down, "weight", [(f"l{i}.mlp.down", (D, mlp["ff"]))]),
                         TensorBinding(ffn, "act", [(f"l{i}.mlp.act", (4,))])]
            norm2 = _norm(bindings, f"l{i}.norm2", D, eps, norm_init)
            norm2b = _norm(bindings, f"l{i}.norm2b", D, eps, norm_init)
        blocks.append(BLOCKS.build("sandwich", norm1=norm1, mixer=mixer, norm1b=norm1b, norm2=norm2, ffn=ffn, norm2b=norm2b))
    n = len(cfg.layers)
    extras, order = [], []
    if cfg.has_loop:
        entry = LoopEntry(D, cfg.loop_times, source=keep)
        extras.append(("loop", entry))
        bindings += [TensorBinding(entry.inp, "weight", [("loop.in", (D, 2 * D))]),
                     TensorBinding(entry, "step", [("loop.step", (cfg.loop_times, D))])]
        order += [LayerCall(i) for i in range(cfg.loop_start)]
        for t in range(cfg.loop_times):
            order += [LayerCall(i, enter=(entry, t) if i == cfg.loop_start else None)
                      for i in range(cfg.loop_start, cfg.loop_stop)]
        order += [LayerCall(i) for i in range(cfg.loop_stop, n)]
    else:
        order = [LayerCall(i) for i in range(n)]
    final_norm = _norm(bindings, "final.norm", D, eps, norm_init)
    head = LMHead(D, cfg.vocab, softcap=cfg.logit_softcap)
    bindings.append(TensorBinding(head, "weight", [("head", (cfg.vocab, D))]))
    return ModelSpec(cfg, embedding, blocks, order, final_norm, head, bindings, extras=extras)


register_architecture("Rivetar", RivetarConfig, build_rivetar, replace=True)
