"""Typed model configuration read from an architecture's own ``config.json`` keys.

The reference keeps the same facts in a 64-byte binary header (``src/model/weights.cpp:24-40``)
that its export script fills from the HF config (``tools/export_weights.py:59-67``); here the
JSON is read directly.  Every size and constant a layer needs comes from this object: parts
take them as constructor parameters and never read a config themselves.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields, asdict
from typing import Any, Dict, Optional


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model: names the key and the reason."""


def _require(d: Dict[str, Any], key: str, typ, where: str):
    if key not in d or d[key] is None:
        raise ConfigError(f"{where}: required key '{key}' is missing")
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"{where}: key '{key}' must be an integer, got {v!r}")
    elif typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{where}: key '{key}' must be a number, got {v!r}")
        v = float(v)
    return v


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration; subclasses add their own keys."""
    architecture: str

    def to_json_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    """Llama dense decoder (``LlamaForCausalLM``).

    Field <- config.json key, as the reference maps them (``src/model/weights.h:12-18``,
    ``tools/export_weights.py:59-67``).  ``head_dim`` is the key of that name when present and
    ``hidden_size // num_attention_heads`` otherwise (the reference computes the latter at
    export, ``tools/export_weights.py:62``); it need not equal ``hidden_size / heads`` here.
    """
    vocab_size: int = 0
    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    max_position_embeddings: int = 0
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"

    # ---- derived sizes
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    def validate(self) -> None:
        w = "LlamaConfig"
        for f in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                  "num_attention_heads", "num_key_value_heads", "head_dim",
                  "max_position_embeddings"):
            if getattr(self, f) <= 0:
                raise ConfigError(f"{w}: '{f}' must be positive, got {getattr(self, f)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"{w}: num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"{w}: head_dim ({self.head_dim}) must be even for rotary pairs")
        if self.hidden_act != "silu":
            raise ConfigError(f"{w}: hidden_act '{self.hidden_act}' is not supported (only 'silu')")
        if not (self.rope_theta > 0):
            raise ConfigError(f"{w}: rope_theta must be positive, got {self.rope_theta}")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"{w}: rms_norm_eps must be positive, got {self.rms_norm_eps}")

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        w = "config.json (LlamaForCausalLM)"
        heads = _require(d, "num_attention_heads", int, w)
        hidden = _require(d, "hidden_size", int, w)
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"{w}: hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads} and no 'head_dim' is given")
            head_dim = hidden // heads
        # rotary base: plain key, or the nested form newer exports use
        rope_params = d.get("rope_parameters") or {}
        theta = d.get("rope_theta", rope_params.get("rope_theta", 10000.0))
        scaling = d.get("rope_scaling")
        if scaling is None and rope_params.get("rope_type", "default") not in ("default", None):
            scaling = rope_params
        if scaling not in (None, {}):
            rt = scaling.get("rope_type", scaling.get("type", "?")) if isinstance(scaling, dict) else scaling
            if rt != "default":
                raise ConfigError(f"{w}: rope scaling '{rt}' is not supported (plain rotary only)")
        for key in ("attention_bias", "mlp_bias"):
            if d.get(key):
                raise ConfigError(f"{w}: '{key}' = true is not supported (no bias tensors)")
        if d.get("sliding_window") not in (None, 0):
            raise ConfigError(f"{w}: 'sliding_window' is not part of this architecture")
        cfg = cls(
            architecture="LlamaForCausalLM",
            vocab_size=_require(d, "vocab_size", int, w),
            hidden_size=hidden,
            intermediate_size=_require(d, "intermediate_size", int, w),
            num_hidden_layers=_require(d, "num_hidden_layers", int, w),
            num_attention_heads=heads,
            num_key_value_heads=int(d.get("num_key_value_heads") or heads),
            head_dim=int(head_dim),
            max_position_embeddings=_require(d, "max_position_embeddings", int, w),
            rope_theta=float(theta),
            rms_norm_eps=_require(d, "rms_norm_eps", float, w),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            hidden_act=str(d.get("hidden_act", "silu")),
        )
        cfg.validate()
        return cfg

    def to_json_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d.pop("architecture")
        d["architectures"] = [self.architecture]
        d["model_type"] = "llama"
        return d


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in model folder '{folder}'")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return d


# ------------------------------------------------------------------------------------ Tolanex

def _section(d: Dict[str, Any], key: str, where: str, optional: bool = False) -> Optional[Dict[str, Any]]:
    v = d.get(key)
    if v is None:
        if optional:
            return None
        raise ConfigError(f"{where}: required section '{key}' is missing")
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: '{key}' must be an object, got {v!r}")
    return v


@dataclass(frozen=True)
class TolanexConfig(ModelConfig):
    """Tolanex: a decoder whose layers are listed one by one in config.json.

    Top level: ``vocab``, ``width``, ``max_positions`` (rows of the learned position table),
    ``norm.eps``, ``residual_mult``, ``embedding.bigram`` {buckets, mul_prev, mul_cur} (optional) and
    ``layers``: a list of {type, mixer, mlp}.  ``type`` "delta": mixer {heads, kv_heads, dim, vdim,
    conv}; "latent_attention": mixer {heads, dim, vdim, kv_rank, scale, kv_from (optional: the layer
    whose cached latent this one reads)}.  ``mlp`` is null or {kind: "moe", expert.ff, router
    {experts, top, scale, groups {count, keep}}, shared {ff} (optional)}.  ``layers`` is kept as the
    parsed JSON (a tuple of dicts) after validation; the builder reads every size from it."""
    vocab: int = 0
    width: int = 0
    max_positions: int = 0
    norm_eps: float = 1e-6
    residual_mult: float = 1.0
    bigram_buckets: int = 0
    bigram_mul_prev: int = 0
    bigram_mul_cur: int = 0
    layers: tuple = ()

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any]) -> "TolanexConfig":
        w = "config.json (Tolanex)"
        norm = _section(d, "norm", w)
        emb = _section(d, "embedding", w, optional=True) or {}
        big = _section(emb, "bigram", w + " embedding", optional=True)
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{w}: 'layers' must be a non-empty list")
        cfg = cls(
            architecture="Tolanex",
            vocab=_require(d, "vocab", int, w),
            width=_require(d, "width", int, w),
            max_positions=int(d.get("max_positions") or 0),
            norm_eps=_require(norm, "eps", float, w + " norm"),
            residual_mult=float(d.get("residual_mult", 1.0)),
            bigram_buckets=_require(big, "buckets", int, w + " bigram") if big else 0,
            bigram_mul_prev=_require(big, "mul_prev", int, w + " bigram") if big else 0,
            bigram_mul_cur=_require(big, "mul_cur", int, w + " bigram") if big else 0,
            layers=tuple(json.loads(json.dumps(layers))),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        w = "TolanexConfig"
        for f in ("vocab", "width"):
            if getattr(self, f) <= 0:
                raise ConfigError(f"{w}: '{f}' must be positive, got {getattr(self, f)}")
        if self.max_positions < 0 or self.bigram_buckets < 0:
            raise ConfigError(f"{w}: 'max_positions' and 'bigram.buckets' cannot be negative")
        if not (self.norm_eps > 0):
            raise ConfigError(f"{w}: norm.eps must be positive, got {self.norm_eps}")
        for i, layer in enumerate(self.layers):
            lw = f"{w}: layer {i}"
            if not isinstance(layer, dict):
                raise ConfigError(f"{lw} must be an object")
            kind = layer.get("type")
            m = _section(layer, "mixer", lw)
            if kind == "delta":
                for k in ("heads", "kv_heads", "dim", "vdim", "conv"):
                    if _require(m, k, int, lw + " mixer") <= 0:
                        raise ConfigError(f"{lw}: mixer.{k} must be positive")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{lw}: mixer.heads ({m['heads']}) must be a multiple of mixer.kv_heads ({m['kv_heads']})")
            elif kind == "latent_attention":
                for k in ("heads", "dim", "vdim", "kv_rank"):
                    if _require(m, k, int, lw + " mixer") <= 0:
                        raise ConfigError(f"{lw}: mixer.{k} must be positive")
                _require(m, "scale", float, lw + " mixer")
                src = m.get("kv_from")
                if src is not None:
                    ok = isinstance(src, int) and 0 <= src < i and self.layers[src].get("type") == "latent_attention" \
                        and self.layers[src]["mixer"].get("kv_from") is None \
                        and self.layers[src]["mixer"].get("kv_rank") == m["kv_rank"]
                    if not ok:
                        raise ConfigError(f"{lw}: mixer.kv_from = {src!r} must name an earlier latent_attention layer "
                                          f"with a latent of its own and the same kv_rank")
            else:
                raise ConfigError(f"{lw}: unknown type {kind!r} (known: delta, latent_attention)")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                raise ConfigError(f"{lw}: mlp must be null or of kind 'moe', got {mlp!r}")
            if _require(_section(mlp, "expert", lw + " mlp"), "ff", int, lw + " mlp.expert") <= 0:
                raise ConfigError(f"{lw}: mlp.expert.ff must be positive")
            r = _section(mlp, "router", lw + " mlp")
            experts, top = _require(r, "experts", int, lw + " router"), _require(r, "top", int, lw + " router")
            groups = _section(r, "groups", lw + " router", optional=True) or {"count": 1, "keep": 1}
            count, keep = _require(groups, "count", int, lw + " groups"), _require(groups, "keep", int, lw + " groups")
            if experts <= 0 or count <= 0 or experts % count or not (1 <= keep <= count) \
                    or not (1 <= top <= experts // count * keep):
                raise ConfigError(f"{lw}: router cannot choose {top} of {experts} experts in {count} groups of which {keep} are kept")
            shared = _section(mlp, "shared", lw + " mlp", optional=True)
            if shared is not None and _require(shared, "ff", int, lw + " mlp.shared") <= 0:
                raise ConfigError(f"{lw}: mlp.shared.ff must be positive")

    def to_json_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                             "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
                             "residual_mult": self.residual_mult, "layers": json.loads(json.dumps(list(self.layers)))}
        if self.bigram_buckets:
            d["embedding"] = {"bigram": {"buckets": self.bigram_buckets, "mul_prev": self.bigram_mul_prev,
                                         "mul_cur": self.bigram_mul_cur}}
        return d


# ------------------------------------------------------------------------------------ Bifatar

def _positive_ints(m: Dict[str, Any], keys, where: str) -> None:
    for k in keys:
        if _require(m, k, int, where) <= 0:
            raise ConfigError(f"{where}: '{k}' must be positive")


def _check_rot(m: Dict[str, Any], where: str) -> None:
    rot = _section(m, "rot", where, optional=True)
    if rot is None:
        return
    dims = _require(rot, "dims", int, where + " rot")
    if _require(rot, "base", float, where + " rot") <= 0 or dims <= 0 or dims % 2 or dims > m["dim"]:
        raise ConfigError(f"{where}: rot needs a positive base and an even 'dims' within 'dim', got {rot!r}")


def _check_heads(m: Dict[str, Any], where: str) -> None:
    _positive_ints(m, ("heads", "kv_heads", "dim", "vdim"), where)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}: heads ({m['heads']}) must be a multiple of kv_heads ({m['kv_heads']})")


@dataclass(frozen=True)
class BifatarConfig(ModelConfig):
    """Bifatar: a decoder whose layers are listed one by one; every layer is a parallel block
    (one tanh norm, mixer and feed-forward read its output, their sum joins the stream).

    Top level: ``vocab``, ``width``, ``norm.eps`` and ``layers``: a list of {type, mixer, mlp}.
    ``type`` "attention": mixer {heads, kv_heads, dim, vdim, scale, rot {base, dims} (optional), mask {size}
    (optional), softcap (optional), v_mix (optional)}; "mamba2": mixer {heads, vdim, state, groups, conv,
    norm_groups}; "parallel": mixer {left {heads, kv_heads, dim, vdim, scale, rot (optional)}, right {heads,
    kv_heads, dim, vdim, conv}, left_scale, right_scale}.  ``mlp`` is null or {kind: "dense", ff}.
    ``layers`` is kept as the parsed JSON after validation; the builder reads every size from it (and the
    ranks of the right mixer's two-stage projections from the checkpoint's shapes, see the builder)."""
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    layers: tuple = ()

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any]) -> "BifatarConfig":
        w = "config.json (Bifatar)"
        norm = _section(d, "norm", w)
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{w}: 'layers' must be a non-empty list")
        cfg = cls(architecture="Bifatar", vocab=_require(d, "vocab", int, w), width=_require(d, "width", int, w),
                  norm_eps=_require(norm, "eps", float, w + " norm"), layers=tuple(json.loads(json.dumps(layers))))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        w = "BifatarConfig"
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"{w}: 'vocab' and 'width' must be positive")
        if not (self.norm_eps > 0):
            raise ConfigError(f"{w}: norm.eps must be positive, got {self.norm_eps}")
        mixed = None
        for i, layer in enumerate(self.layers):
            lw = f"{w}: layer {i}"
            if not isinstance(layer, dict):
                raise ConfigError(f"{lw} must be an object")
            kind = layer.get("type")
            m = _section(layer, "mixer", lw)
            mw = lw + " mixer"
            if kind == "attention":
                _check_heads(m, mw)
                _require(m, "scale", float, mw)
                _check_rot(m, mw)
                mask = _section(m, "mask", mw, optional=True)
                if mask is not None and _require(mask, "size", int, mw + " mask") <= 0:
                    raise ConfigError(f"{mw}: mask.size must be positive")
                if m.get("softcap") is not None and not (_require(m, "softcap", float, mw) > 0):
                    raise ConfigError(f"{mw}: softcap must be positive")
                if m.get("v_mix"):
                    shape = (m["kv_heads"], m["vdim"])
                    if mixed is not None and mixed != shape:
                        raise ConfigError(f"{mw}: layers that mix values need the same kv_heads and vdim as the first of them")
                    mixed = shape
            elif kind == "mamba2":
                _positive_ints(m, ("heads", "vdim", "state", "groups", "conv", "norm_groups"), mw)
                if m["heads"] % m["groups"] or (m["heads"] * m["vdim"]) % m["norm_groups"]:
                    raise ConfigError(f"{mw}: heads must be a multiple of groups and heads*vdim of norm_groups")
            elif kind == "parallel":
                left, right = _section(m, "left", mw), _section(m, "right", mw)
                _check_heads(left, mw + ".left")
                _require(left, "scale", float, mw + ".left")
                _check_rot(left, mw + ".left")
                _check_heads(right, mw + ".right")
                _positive_ints(right, ("conv",), mw + ".right")
                _require(m, "left_scale", float, mw)
                _require(m, "right_scale", float, mw)
            else:
                raise ConfigError(f"{lw}: unknown type {kind!r} (known: attention, mamba2, parallel)")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                raise ConfigError(f"{lw}: mlp must be null or of kind 'dense', got {mlp!r}")
            if _require(mlp, "ff", int, lw + " mlp") <= 0:
                raise ConfigError(f"{lw}: mlp.ff must be positive")

    def to_json_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": json.loads(json.dumps(list(self.layers)))}


@dataclass(frozen=True)
class RivetarConfig(ModelConfig):
    """Rivetar: a decoder whose layers are listed one by one, every sublayer normalised on both sides
    (x += norm_b(sublayer(norm(x))), the norms' weights stored as their distance from one), with a span of
    layers that runs several times in a row.

    Top level: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``logit_softcap`` (optional, > 0),
    ``loop`` {start, stop, times} (optional) and ``layers``: a list of {type, mixer, mlp}.
    ``type`` "latent_attention": mixer {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot {base, dims}};
    "attention": mixer {heads, kv_heads, dim, vdim, scale, rot {base, dims}, mask {size, keep_first} (optional)};
    "gla": mixer {heads, dim, vdim, tau}.  ``mlp`` is null or {kind: "dense", ff}.
    ``layers`` is kept as the parsed JSON after validation; the builder reads every size from it (the rank
    of the decay's two-stage projection comes from the checkpoint's shapes, or from mixer key ``decay_rank``
    when a model is made without a checkpoint)."""
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    logit_softcap: float = 0.0
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    layers: tuple = ()

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any]) -> "RivetarConfig":
        w = "config.json (Rivetar)"
        norm = _section(d, "norm", w)
        emb = _section(d, "embedding", w, optional=True) or {}
        loop = _section(d, "loop", w, optional=True)
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{w}: 'layers' must be a non-empty list")
        cap = d.get("logit_softcap")
        cfg = cls(architecture="Rivetar", vocab=_require(d, "vocab", int, w), width=_require(d, "width", int, w),
                  norm_eps=_require(norm, "eps", float, w + " norm"),
                  embedding_scale=_require(emb, "scale", float, w + " embedding") if "scale" in emb else 1.0,
                  logit_softcap=_require(d, "logit_softcap", float, w) if cap is not None else 0.0,
                  loop_start=_require(loop, "start", int, w + " loop") if loop else 0,
                  loop_stop=_require(loop, "stop", int, w + " loop") if loop else 0,
                  loop_times=_require(loop, "times", int, w + " loop") if loop else 1,
                  layers=tuple(json.loads(json.dumps(layers))))
        cfg.validate()
        return cfg

    @property
    def has_loop(self) -> bool:
        return self.loop_stop > self.loop_start

    def validate(self) -> None:
        w = "RivetarConfig"
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"{w}: 'vocab' and 'width' must be positive")
        if not (self.norm_eps > 0):
            raise ConfigError(f"{w}: norm.eps must be positive, got {self.norm_eps}")
        if self.logit_softcap < 0:
            raise ConfigError(f"{w}: logit_softcap must be positive when given")
        n = len(self.layers)
        if self.loop_stop or self.loop_start or self.loop_times != 1:
            if not (0 <= self.loop_start < self.loop_stop <= n) or self.loop_times < 1:
                raise ConfigError(f"{w}: loop needs 0 <= start < stop <= {n} layers and times >= 1, got "
                                  f"start {self.loop_start}, stop {self.loop_stop}, times {self.loop_times}")
        for i, layer in enumerate(self.layers):
            lw = f"{w}: layer {i}"
            if not isinstance(layer, dict):
                raise ConfigError(f"{lw} must be an object")
            kind = layer.get("type")
            m = _section(layer, "mixer", lw)
            mw = lw + " mixer"
            if kind == "latent_attention":
                _positive_ints(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"), mw)
                _require(m, "scale", float, mw)
                rot = _section(m, "rot", mw)
                dims = _require(rot, "dims", int, mw + " rot")
                if _require(rot, "base", float, mw + " rot") <= 0 or dims <= 0 or dims % 2 or dims > m["rot_dim"]:
                    raise ConfigError(f"{mw}: rot needs a positive base and an even 'dims' within 'rot_dim', got {rot!r}")
            elif kind == "attention":
                _check_heads(m, mw)
                _require(m, "scale", float, mw)
                _section(m, "rot", mw)
                _check_rot(m, mw)
                if m["vdim"] % 2:
                    raise ConfigError(f"{mw}: values turn in pairs, 'vdim' must be even")
                mask = _section(m, "mask", mw, optional=True)
                if mask is not None:
                    if _require(mask, "size", int, mw + " mask") <= 0:
                        raise ConfigError(f"{mw}: mask.size must be positive")
                    if mask.get("keep_first") is not None and _require(mask, "keep_first", int, mw + " mask") < 0:
                        raise ConfigError(f"{mw}: mask.keep_first must not be negative")
            elif kind == "gla":
                _positive_ints(m, ("heads", "dim", "vdim"), mw)
                if not (_require(m, "tau", float, mw) > 0):
                    raise ConfigError(f"{mw}: tau must be positive")
            else:
                raise ConfigError(f"{lw}: unknown type {kind!r} (known: attention, gla, latent_attention)")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                raise ConfigError(f"{lw}: mlp must be null or of kind 'dense', got {mlp!r}")
            if _require(mlp, "ff", int, lw + " mlp") <= 0:
                raise ConfigError(f"{lw}: mlp.ff must be positive")

    def to_json_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
             "layers": json.loads(json.dumps(list(self.layers)))}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        if self.has_loop:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return d


# ------------------------------------------------------------------------------------ Lobutar

@dataclass(frozen=True)
class LobutarConfig(ModelConfig):
    """Lobutar: a decoder whose layers are listed one by one, pre-norm layers over ``streams`` residual streams
    (hyper-connections), a layer optionally running with an earlier layer's weights.

    Top level: ``vocab``, ``width``, ``norm.eps``, ``streams`` and ``layers``: a list of {type, mixer, mlp, weights_of}.
    ``type`` "attention" (differential attention): mixer {heads, kv_heads, dim, vdim, diff, scale, rot {base, dims}};
    "latent_attention": mixer {heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}, mask {size} (optional)}.
    ``mlp`` is null, {kind: "dense", ff} or {kind: "moe", expert {ff}, router {experts, top, scale, groups {count, keep}},
    shared {ff} (optional)}.  ``weights_of``: j (optional): the layer has no tensors of its own and runs with layer j's
    parts (its entry otherwise repeats layer j's, whose sizes and constants are the ones used; j may itself name an
    earlier layer).  ``layers`` is kept as the parsed JSON after validation; the builder reads
    every size from it."""
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    streams: int = 1
    layers: tuple = ()

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any]) -> "LobutarConfig":
        w = "config.json (Lobutar)"
        norm = _section(d, "norm", w)
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{w}: 'layers' must be a non-empty list")
        cfg = cls(architecture="Lobutar", vocab=_require(d, "vocab", int, w), width=_require(d, "width", int, w),
                  norm_eps=_require(norm, "eps", float, w + " norm"), streams=_require(d, "streams", int, w),
                  layers=tuple(json.loads(json.dumps(layers))))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        w = "LobutarConfig"
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError(f"{w}: 'vocab' and 'width' must be positive")
        if not (self.norm_eps > 0):
            raise ConfigError(f"{w}: norm.eps must be positive, got {self.norm_eps}")
        if not (1 <= self.streams <= 16):
            raise ConfigError(f"{w}: 'streams' must lie in 1..16, got {self.streams}")
        for i, layer in enumerate(self.layers):
            lw = f"{w}: layer {i}"
            if not isinstance(layer, dict):
                raise ConfigError(f"{lw} must be an object")
            src = layer.get("weights_of")
            if src is not None:
                if isinstance(src, bool) or not isinstance(src, int) or not (0 <= src < i):
                    raise ConfigError(f"{lw}: weights_of must name an earlier layer, got {src!r}")
                if layer.get("type") != self.layers[src].get("type"):
                    raise ConfigError(f"{lw}: a layer that runs with layer {src}'s weights must have the same type")
            kind = layer.get("type")
            m = _section(layer, "mixer", lw)
            mw = lw + " mixer"
            if kind == "attention":
                _check_heads(m, mw)
                _require(m, "scale", float, mw)
                _require(m, "diff", float, mw)
                _check_rot(m, mw)
            elif kind == "latent_attention":
                _positive_ints(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank"), mw)
                _require(m, "scale", float, mw)
                rot = _section(m, "rot", mw)
                dims = _require(rot, "dims", int, mw + " rot")
                if _require(rot, "base", float, mw + " rot") <= 0 or dims <= 0 or dims % 2 or dims > m["rot_dim"]:
                    raise ConfigError(f"{mw}: rot needs a positive base and an even 'dims' within 'rot_dim', got {rot!r}")
                mask = _section(m, "mask", mw, optional=True)
                if mask is not None and _require(mask, "size", int, mw + " mask") <= 0:
                    raise ConfigError(f"{mw}: mask.size must be positive")
            else:
                raise ConfigError(f"{lw}: unknown type {kind!r} (known: attention, latent_attention)")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            pw = lw + " mlp"
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                raise ConfigError(f"{lw}: mlp must be null or of kind 'dense' or 'moe', got {mlp!r}")
            if mlp["kind"] == "dense":
                _positive_ints(mlp, ("ff",), pw)
                continue
            _positive_ints(_section(mlp, "expert", pw), ("ff",), pw + " expert")
            r = _section(mlp, "router", pw)
            _positive_ints(r, ("experts", "top"), pw + " router")
            if "scale" in r:
                _require(r, "scale", float, pw + " router")
            g = _section(r, "groups", pw + " router", optional=True)
            count, keep = 1, 1
            if g is not None:
                _positive_ints(g, ("count", "keep"), pw + " router groups")
                count, keep = g["count"], g["keep"]
            if r["experts"] % count or keep > count or r["top"] > (r["experts"] // count) * keep:
                raise ConfigError(f"{pw}: {r['experts']} experts in {count} groups of which {keep} are kept cannot give {r['top']} choices")
            shared = _section(mlp, "shared", pw, optional=True)
            if shared is not None:
                _positive_ints(shared, ("ff",), pw + " shared")

    def to_json_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "streams": self.streams, "layers": json.loads(json.dumps(list(self.layers)))}
