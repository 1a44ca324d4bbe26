"""Topunex: a decoder whose ``config.json`` lists its layers one by one, each normed only behind its sublayers.

A layer is  x += norm1(mixer(x)); x += norm2(ff(x)): the sublayers read the stream itself (block kind ``postnorm``).
The typed configuration below reads every key, checks it, and states the model as data for the generic decoder:

  * mixer "attention" -> the general form of mixer kind ``attention``: grouped heads with biased q, k and output
    projections, values that are the projected keys, rotation (rotate-half layout, the first ``rot.dims`` dimensions, with
    the wavelength-dependent rescaling of ``rot.scaling``) followed by a division of q and k by their root mean square,
    capped scores (``softcap``), a sliding window ``mask.size`` below which the first ``mask.keep_first`` keys stay visible,
    a learned sink per head, and a sigmoid gate on the heads from a projection of the mixer's input;
  * ``mlp.kind`` "dense" -> feed-forward kind ``swiglu`` with biases;
  * ``mlp.kind`` "moe" -> feed-forward kind ``moe``: sigmoid router, ``router.top`` of ``router.experts`` clamped gated
    experts weighted by score * ``router.scale`` (not renormalised), plus an optional shared expert (``clamped_glu``);
    the experts' sigmoid slope 1.702 and the + 1 on the clamped up part are the design's;
  * ``mlp`` null -> the layer has its mixer only.

Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.{q,q.b,k,k.b,g,o,o.b,sink}``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.model_config import ConfigError, require
from ..config.registry import register_architecture
from ..config.specs import BlockSpec, FeedForwardSpec, LayerCall, MixerSpec, ModelSpec, NormSpec, PositionSpec

GATE_SLOPE = 1.702              # an expert's g * sigmoid(1.702 g)
UP_SHIFT = 1.0                  # ... * (u + 1)

_ATTENTION_NAMES = (("q", "q"), ("k", "k"), ("o", "o"), ("gate", "g"), ("sinks", "sink"),
                    ("q_bias", "q.b"), ("k_bias", "k.b"), ("o_bias", "o.b"))
_FF_NAMES = (("gate", "gate"), ("up", "up"), ("down", "down"))
_MOE_NAMES = (("router", "router"), ("gate", "gate"), ("up", "up"), ("down", "down"))


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


def _positive_number(raw: Dict[str, Any], key: str, where: str) -> float:
    try:
        value = require(raw, key, float)
    except ConfigError as e:
        raise ConfigError(f"{e} (in {where})") from None
    if not (value > 0.0):
        raise ConfigError(f"config.json: {where}'{key}' must be positive, found {value}")
    return value


def _check_expert(raw: Dict[str, Any], where: str) -> None:
    _positive(raw, "ff", where)
    if raw.get("limit") is not None:
        _positive_number(raw, "limit", where)


@dataclass(frozen=True)
class TopunexConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[Dict[str, Any], ...]          # as config.json lists them, checked
    architecture: str = "Topunex"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "TopunexConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        eps = require(_sub(raw, "norm", ""), "eps", float)
        cfg = cls(vocab=_positive(raw, "vocab", ""), width=_positive(raw, "width", ""), norm_eps=eps,
                  layers=tuple(copy.deepcopy(layers)))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not (self.norm_eps > 0.0):
            raise ConfigError("config.json: norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict) or layer.get("type") != "attention":
                raise ConfigError(f"config.json: {where}type '{layer.get('type') if isinstance(layer, dict) else layer}' is not 'attention'")
            m = _sub(layer, "mixer", where)
            wm = where + "mixer."
            for key in ("heads", "kv_heads", "dim"):
                _positive(m, key, wm)
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"config.json: {wm}heads ({m['heads']}) is not a multiple of kv_heads ({m['kv_heads']})")
            if m.get("vdim") is not None and _positive(m, "vdim", wm) != m["dim"]:
                raise ConfigError(f"config.json: {wm}vdim ({m['vdim']}) must equal dim ({m['dim']}): the values are the keys")
            _positive_number(m, "scale", wm)
            if m.get("softcap") is not None:
                _positive_number(m, "softcap", wm)
            rot = m.get("rot")
            if rot is not None:
                rot = _sub(m, "rot", wm)
                dims = _positive(rot, "dims", wm + "rot.")
                if dims % 2 or dims > m["dim"]:
                    raise ConfigError(f"config.json: {wm}rot.dims ({dims}) must be even and at most dim ({m['dim']})")
                _positive_number(rot, "base", wm + "rot.")
                if rot.get("scaling") is not None:
                    sc = _sub(rot, "scaling", wm + "rot.")
                    for key in ("factor", "low", "high", "original"):
                        _positive_number(sc, key, wm + "rot.scaling.")
                    if not (float(sc["high"]) > float(sc["low"])):
                        raise ConfigError(f"config.json: {wm}rot.scaling: high must exceed low")
            mask = m.get("mask")
            if mask is not None:
                mask = _sub(m, "mask", wm)
                if mask.get("size") is not None:
                    _positive(mask, "size", wm + "mask.")
                keep = mask.get("keep_first", 0)
                if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
                    raise ConfigError(f"config.json: {wm}mask.keep_first must be an integer >= 0")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            wf = where + "mlp."
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                raise ConfigError(f"config.json: {wf}kind must be 'dense' or 'moe' (or mlp null)")
            if mlp["kind"] == "dense":
                _positive(mlp, "ff", wf)
                continue
            _check_expert(_sub(mlp, "expert", wf), wf + "expert.")
            router = _sub(mlp, "router", wf)
            experts, top = _positive(router, "experts", wf + "router."), _positive(router, "top", wf + "router.")
            if top > experts:
                raise ConfigError(f"config.json: {wf}router.top ({top}) exceeds router.experts ({experts})")
            if router.get("scale") is not None:
                require(router, "scale", float)
            if mlp.get("shared") is not None:
                _check_expert(_sub(mlp, "shared", wf), wf + "shared.")

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "layers": copy.deepcopy(list(self.layers))}

    # ------------------------------------------------------------------ the model as data
    def _mixer_spec(self, m: Dict[str, Any]) -> MixerSpec:
        rot, mask = m.get("rot"), m.get("mask") or {}
        position = None
        if rot is not None:
            sc = rot.get("scaling")
            scaling = None if sc is None else tuple(float(sc[k]) for k in ("factor", "low", "high", "original"))
            position = PositionSpec("rope", int(m["dim"]), int(rot["dims"]), float(rot["base"]), scaling)
        return MixerSpec(kind="attention", hidden=self.width, n_heads=int(m["heads"]), n_kv_heads=int(m["kv_heads"]),
                         head_dim=int(m["dim"]), scale=float(m["scale"]),
                         window=None if mask.get("size") is None else int(mask["size"]), keep_first=int(mask.get("keep_first", 0)),
                         softcap=None if m.get("softcap") is None else float(m["softcap"]), position=position,
                         qk_norm_eps=self.norm_eps, qk_norm_weight=False, qk_norm_after_rotation=True, sinks=True, bias=True,
                         output_gate=True, values_from_keys=True, tensor_names=_ATTENTION_NAMES)

    def _feed_forward_spec(self, mlp: Optional[Dict[str, Any]]) -> Optional[FeedForwardSpec]:
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return FeedForwardSpec("swiglu", self.width, int(mlp["ff"]), "silu", extra=(("bias", True), ("tensor_names", _FF_NAMES)))

        def gated(e: Dict[str, Any]) -> Tuple[Tuple[str, object], ...]:
            return (("limit", None if e.get("limit") is None else float(e["limit"])), ("alpha", GATE_SLOPE), ("shift", UP_SHIFT))
        expert, router, shared = mlp["expert"], mlp["router"], mlp.get("shared")
        shared_spec = None
        if shared is not None:
            if shared.get("limit") is None:
                raise ConfigError("config.json: a shared expert needs its limit")
            shared_spec = FeedForwardSpec("clamped_glu", self.width, int(shared["ff"]), "sigmoid",
                                          extra=gated(shared)[:2] + (("tensor_names", _FF_NAMES),))
        return FeedForwardSpec("moe", self.width, int(expert["ff"]), "sigmoid",
                               extra=gated(expert) + (("experts", int(router["experts"])), ("top", int(router["top"])),
                                                      ("router_scale", float(router.get("scale", 1.0) or 1.0)),
                                                      ("renormalize", False), ("shared", shared_spec),
                                                      ("shared_prefix", "shared."), ("tensor_names", _MOE_NAMES)))

    def model_spec(self) -> ModelSpec:
        norm = NormSpec("rmsnorm", self.width, self.norm_eps, suffix="")
        blocks: List[BlockSpec] = []
        for i, layer in enumerate(self.layers):
            ffn = self._feed_forward_spec(layer.get("mlp"))
            blocks.append(BlockSpec(
                kind="postnorm", mixer=self._mixer_spec(layer["mixer"]), feed_forward=ffn, mixer_norm=None, feed_forward_norm=None,
                weight_prefix=f"l{i}.",
                names=(("mixer", "mix."), ("feed_forward", "mlp."), ("mixer_post_norm", "norm1"), ("feed_forward_post_norm", "norm2")),
                mixer_post_norm=norm, feed_forward_post_norm=norm if ffn is not None else None))
        order = tuple(LayerCall(i, i) for i in range(len(blocks)))
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab, hidden=self.width, blocks=tuple(blocks),
                         run_order=order, final_norm=norm, embed_name="embed", final_norm_name="final.norm", head_name="head",
                         tie_word_embeddings=False, init_std=0.05)


@register_architecture("Topunex")
def topunex_config(raw: dict) -> TopunexConfig:
    return TopunexConfig.from_dict(raw)
