"""Configuration of the Fegarax decoder: a list of layers (each names its mixer's sizes and its feed-forward), the number of
residual streams, the embedding's scale and the norm's eps.

Every size and constant comes from ``config.json``; what a part needs is checked here, so that a folder with a missing
or mistyped key is refused before any weight is read.  Optional keys switch a mechanism off when they are absent: no
``streams`` (one plain residual stream), no ``mask`` (every earlier position is seen), no ``rot`` (no rotation), no
``rot.scaling`` (plain frequencies), no ``v_mix``, ``mlp`` null (a layer without feed-forward).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig, eos_ids, optional, require

MIXER_TYPES = ("attention",)
#: positions a sequence may reach where config.json does not say (`max_positions`); nothing in the design depends on it
DEFAULT_MAX_POSITIONS = 1 << 17


def _obj(raw: Dict[str, Any], key: str, where: str, needed: bool = True) -> Optional[Dict[str, Any]]:
    value = raw.get(key)
    if value is None and not needed:
        return None
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {where}`{key}` must be an object")
    return value


def _int(raw: Dict[str, Any], key: str, where: str, least: int = 1) -> int:
    try:
        value = require(raw, key, int)
    except ConfigError as err:
        raise ConfigError(f"config.json: {where}{str(err).replace('config.json: ', '')}") from None
    if value < least:
        raise ConfigError(f"config.json: {where}`{key}` must be at least {least}, got {value}")
    return value


def _num(raw: Dict[str, Any], key: str, where: str, positive: bool = False) -> float:
    try:
        value = require(raw, key, float)
    except ConfigError as err:
        raise ConfigError(f"config.json: {where}{str(err).replace('config.json: ', '')}") from None
    if positive and value <= 0:
        raise ConfigError(f"config.json: {where}`{key}` must be positive, got {value}")
    return value


@dataclass
class FegaraxLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]

    @classmethod
    def parse(cls, raw: Any, index: int) -> "FegaraxLayer":
        where = f"layers[{index}]: "
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: {where}must be an object")
        kind = raw.get("type")
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {where}`type` {kind!r} is not one of {list(MIXER_TYPES)}")
        m = _obj(raw, "mixer", where)
        mixer: Dict[str, Any] = {"heads": _int(m, "heads", where), "kv_heads": _int(m, "kv_heads", where), "dim": _int(m, "dim", where),
                                 "vdim": _int(m, "vdim", where), "scale": _num(m, "scale", where)}
        if mixer["heads"] % mixer["kv_heads"] != 0:
            raise ConfigError(f"config.json: {where}{mixer['heads']} heads cannot share {mixer['kv_heads']} kv heads evenly")
        mask = _obj(m, "mask", where, needed=False)
        mixer["mask"] = {"size": _int(mask, "size", where + "mask: ")} if mask is not None else None
        rot = _obj(m, "rot", where, needed=False)
        mixer["rot"] = None
        if rot is not None:
            r: Dict[str, Any] = {"base": _num(rot, "base", where + "rot: ", True), "dims": _int(rot, "dims", where + "rot: ", 2), "scaling": None}
            if r["dims"] % 2 or r["dims"] > mixer["dim"]:
                raise ConfigError(f"config.json: {where}`rot.dims` {r['dims']} must be even and at most `dim` {mixer['dim']}")
            sc = _obj(rot, "scaling", where + "rot: ", needed=False)
            if sc is not None:
                r["scaling"] = {k: _num(sc, k, where + "rot.scaling: ", True) for k in ("factor", "original", "fast", "slow")}
                if r["base"] <= 1:
                    raise ConfigError(f"config.json: {where}`rot.base` must be above 1 with `rot.scaling`")
            mixer["rot"] = r
        v_mix = m.get("v_mix", False)
        if not isinstance(v_mix, bool):
            raise ConfigError(f"config.json: {where}`v_mix` must be true or false")
        mixer["v_mix"] = v_mix
        mlp = raw.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict):
                raise ConfigError(f"config.json: {where}`mlp` must be an object or null")
            if mlp.get("kind") != "moe":
                raise ConfigError(f"config.json: {where}`mlp.kind` {mlp.get('kind')!r} is not supported (moe)")
            expert, router = _obj(mlp, "expert", where + "mlp: "), _obj(mlp, "router", where + "mlp: ")
            mlp = {"kind": "moe", "expert": {"ff": _int(expert, "ff", where + "mlp.expert: ")},
                   "router": {"experts": _int(router, "experts", where + "mlp.router: "), "top": _int(router, "top", where + "mlp.router: ")}}
            if mlp["router"]["top"] > mlp["router"]["experts"]:
                raise ConfigError(f"config.json: {where}`mlp.router.top` exceeds `mlp.router.experts`")
        return cls(kind, mixer, mlp)

    def to_json_dict(self) -> Dict[str, Any]:
        m = {k: v for k, v in self.mixer.items() if k not in ("mask", "rot", "v_mix")}
        if self.mixer["mask"] is not None:
            m["mask"] = dict(self.mixer["mask"])
        if self.mixer["rot"] is not None:
            rot = {"base": self.mixer["rot"]["base"], "dims": self.mixer["rot"]["dims"]}
            if self.mixer["rot"]["scaling"] is not None:
                rot["scaling"] = dict(self.mixer["rot"]["scaling"])
            m["rot"] = rot
        if self.mixer["v_mix"]:
            m["v_mix"] = True
        mlp = None
        if self.mlp is not None:
            mlp = {"kind": "moe", "expert": dict(self.mlp["expert"]), "router": dict(self.mlp["router"])}
        return {"type": self.type, "mixer": m, "mlp": mlp}


@dataclass
class FegaraxConfig(ModelConfig):
    layers: List[FegaraxLayer] = field(default_factory=list)
    #: copies of the residual stream (hyper-connections); None: one plain residual stream without their tensors
    streams: Optional[int] = None
    embedding_scale: float = 1.0
    norm_eps: float = 0.0

    ARCHITECTURE = "Fegarax"
    MODEL_TYPE = "fegarax"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], generation: Optional[Dict[str, Any]] = None) -> "FegaraxConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: `layers` must be a non-empty list")
        layers = [FegaraxLayer.parse(layer, i) for i, layer in enumerate(layers_raw)]
        norm = _obj(raw, "norm", "")
        emb = _obj(raw, "embedding", "", needed=False)
        streams = None
        if raw.get("streams") is not None:
            streams = _int(raw, "streams", "")
            if streams > 8:
                raise ConfigError(f"config.json: `streams` {streams} is more than the 8 the kernels are written for")
        eos = eos_ids(raw.get("eos_token_id"))
        if generation is not None and generation.get("eos_token_id") is not None:
            eos = eos_ids(generation.get("eos_token_id"))
        return cls(architecture=cls.ARCHITECTURE, model_type=cls.MODEL_TYPE, vocab_size=_int(raw, "vocab", ""),
                   hidden_size=_int(raw, "width", ""),
                   max_position_embeddings=optional(raw, "max_positions", int, DEFAULT_MAX_POSITIONS),
                   eos_token_ids=eos, raw=dict(raw), layers=layers, streams=streams,
                   embedding_scale=_num(emb, "scale", "embedding: ") if emb is not None and emb.get("scale") is not None else 1.0,
                   norm_eps=_num(norm, "eps", "norm: "))

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
                               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                               "layers": [layer.to_json_dict() for layer in self.layers]}
        if self.streams is not None:
            out["streams"] = self.streams
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_position_embeddings
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
