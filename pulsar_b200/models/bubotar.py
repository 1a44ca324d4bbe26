"""Bubotar: a decoder whose ``config.json`` lists its layers one by one.

Every layer names its mixer ("latent_attention", "mamba1" or "attention") with the mixer's sizes and an optional
feed-forward; a layer is normed before and behind each sublayer.  The typed configuration below reads every key,
checks it, and states the model as data for the generic decoder:

  * "latent_attention" -> mixer kind ``latent_attention``: rotation of neighbouring pairs on the rotated parts, causal,
    an output gate; a layer with ``kv_from: j`` has no down projection and runs against layer j's cache entry;
  * "mamba1" -> mixer kind ``selective_scan``;
  * "attention" -> the general form of mixer kind ``attention``: grouped heads without rotation, the score loses
    2^(-8 (h+1) / heads) * distance (the 8 is the design's), optional chunk mask ``mask.size``;
  * ``mlp.kind`` "dense" -> feed-forward kind ``clamped_glu`` with the design's sigmoid slope 1.702.

Tensor names: ``embed``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.model_config import ConfigError, require
from ..config.registry import register_architecture
from ..config.specs import (BlockSpec, FeedForwardSpec, LayerCall, MixerSpec, ModelSpec, NormSpec, PositionSpec)

DISTANCE_BIAS_RATE = 8.0        # slope of head h: 2^(-8 (h+1) / heads)
GATE_SLOPE = 1.702              # the feed-forward's g * sigmoid(1.702 g)

_LATENT_NAMES = (("q", "q"), ("down", "dkv"), ("latent_norm", "dkv.norm"), ("up_k", "uk"), ("up_v", "uv"), ("gate", "g"), ("o", "o"))
_SCAN_NAMES = (("in", "in"), ("conv", "conv"), ("conv_bias", "conv.b"), ("x", "x"), ("dt", "dt"), ("dt_bias", "dt.b"),
               ("a_log", "A_log"), ("d", "D"), ("o", "o"))
_ATTENTION_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"))
_FF_NAMES = (("gate", "gate"), ("up", "up"), ("down", "down"))


def _sub(raw: Dict[str, Any], key: str, where: str) -> Dict[str, Any]:
    value = raw.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return value


def _positive(raw: Dict[str, Any], key: str, where: str) -> int:
    try:
        value = require(raw, key, int)
    except ConfigError as e:
        raise ConfigError(f"{e} (in {where})") from None
    if value <= 0:
        raise ConfigError(f"config.json: {where}'{key}' must be positive, found {value}")
    return value


@dataclass(frozen=True)
class BubotarConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    layers: Tuple[Dict[str, Any], ...]          # as config.json lists them, checked
    architecture: str = "Bubotar"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "BubotarConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        eps = require(_sub(raw, "norm", ""), "eps", float)
        cfg = cls(vocab=_positive(raw, "vocab", ""), width=_positive(raw, "width", ""), norm_eps=eps,
                  logit_scale=float(raw.get("logit_scale", 1.0)), layers=tuple(copy.deepcopy(layers)))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not (self.norm_eps > 0.0):
            raise ConfigError("config.json: norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            kind = layer.get("type")
            m = _sub(layer, "mixer", where)
            where_m = where + "mixer."
            if kind == "latent_attention":
                for key in ("heads", "dim", "vdim", "kv_rank", "rot_dim"):
                    _positive(m, key, where_m)
                require(m, "scale", float)
                rot = _sub(m, "rot", where_m)
                dims = _positive(rot, "dims", where_m + "rot.")
                if dims % 2 or dims > m["rot_dim"] or not (require(rot, "base", float) > 0.0):
                    raise ConfigError(f"config.json: {where_m}rot: dims must be even and at most rot_dim, base positive")
                src = m.get("kv_from")
                if src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not (0 <= src < i):
                        raise ConfigError(f"config.json: {where_m}kv_from must name an earlier layer")
                    other = self.layers[src]
                    om = other.get("mixer", {})
                    if other.get("type") != "latent_attention" or om.get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where_m}kv_from = {src}: that layer has no latent of its own")
                    if any(om.get(k) != m.get(k) for k in ("kv_rank", "rot_dim", "rot")):
                        raise ConfigError(f"config.json: {where_m}kv_from = {src}: kv_rank, rot_dim and rot must be equal")
            elif kind == "mamba1":
                for key in ("inner", "state", "dt_rank", "conv"):
                    _positive(m, key, where_m)
            elif kind == "attention":
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _positive(m, key, where_m)
                require(m, "scale", float)
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"config.json: {where_m}heads ({m['heads']}) is not a multiple of kv_heads ({m['kv_heads']})")
                if m.get("mask") is not None:
                    _positive(_sub(m, "mask", where_m), "size", where_m + "mask.")
            else:
                raise ConfigError(f"config.json: {where}type '{kind}' is not one of latent_attention, mamba1, attention")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind must be 'dense' (or mlp null)")
                _positive(mlp, "ff", where + "mlp.")
                if not (require(mlp, "limit", float) > 0.0):
                    raise ConfigError(f"config.json: {where}mlp.limit must be positive")

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "logit_scale": self.logit_scale, "layers": copy.deepcopy(list(self.layers))}

    # ------------------------------------------------------------------ the model as data
    def _mixer_spec(self, layer: Dict[str, Any]) -> MixerSpec:
        m, kind = layer["mixer"], layer["type"]
        if kind == "latent_attention":
            position = PositionSpec("rope", int(m["rot_dim"]), int(m["rot"]["dims"]), float(m["rot"]["base"]))
            return MixerSpec(kind="latent_attention", hidden=self.width, n_heads=int(m["heads"]), n_kv_heads=1,
                             head_dim=int(m["dim"]), v_head_dim=int(m["vdim"]), scale=float(m["scale"]), position=position,
                             own_kv=m.get("kv_from") is None, tensor_names=_LATENT_NAMES,
                             extra=(("kv_rank", int(m["kv_rank"])), ("rot_dim", int(m["rot_dim"])),
                                    ("latent_norm_eps", self.norm_eps), ("gated", True)))
        if kind == "mamba1":
            return MixerSpec(kind="selective_scan", hidden=self.width, tensor_names=_SCAN_NAMES,
                             extra=tuple((k, int(m[k])) for k in ("inner", "state", "dt_rank", "conv")))
        mask = m.get("mask")
        return MixerSpec(kind="attention", hidden=self.width, n_heads=int(m["heads"]), n_kv_heads=int(m["kv_heads"]),
                         head_dim=int(m["dim"]), v_head_dim=int(m["vdim"]), scale=float(m["scale"]),
                         chunk=None if mask is None else int(mask["size"]), distance_bias=DISTANCE_BIAS_RATE,
                         tensor_names=_ATTENTION_NAMES)

    def model_spec(self) -> ModelSpec:
        norm = NormSpec("rmsnorm", self.width, self.norm_eps, suffix="")
        blocks: List[BlockSpec] = []
        order: List[LayerCall] = []
        entry_of: Dict[int, int] = {}
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            ffn = None
            if mlp is not None:
                ffn = FeedForwardSpec("clamped_glu", self.width, int(mlp["ff"]), "sigmoid",
                                      extra=(("limit", float(mlp["limit"])), ("alpha", GATE_SLOPE), ("tensor_names", _FF_NAMES)))
            blocks.append(BlockSpec(
                kind="sandwich", mixer=self._mixer_spec(layer), feed_forward=ffn, mixer_norm=norm,
                feed_forward_norm=norm if ffn is not None else None, weight_prefix=f"l{i}.",
                names=(("mixer", "mix."), ("feed_forward", "mlp."), ("mixer_norm", "norm1"), ("mixer_post_norm", "norm1b"),
                       ("feed_forward_norm", "norm2"), ("feed_forward_post_norm", "norm2b")),
                mixer_post_norm=norm, feed_forward_post_norm=norm if ffn is not None else None))
            src = layer["mixer"].get("kv_from") if layer["type"] == "latent_attention" else None
            if src is None:
                entry_of[i] = len(entry_of)
                order.append(LayerCall(i, entry_of[i]))
            else:
                order.append(LayerCall(i, entry_of[src]))
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab, hidden=self.width, blocks=tuple(blocks),
                         run_order=tuple(order), final_norm=norm, embed_name="embed", final_norm_name="final.norm",
                         head_name="head", tie_word_embeddings=False, init_std=0.05, logit_scale=self.logit_scale)


@register_architecture("Bubotar")
def bubotar_config(raw: dict) -> BubotarConfig:
    return BubotarConfig.from_dict(raw)
