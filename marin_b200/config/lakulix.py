"""Configuration of the Lakulix decoder: a list of layers that differ from one another (each names its mixer, the mixer's
sizes and its feed-forward), a loop over a run of layers, and a few constants of the whole model.

Every size and constant comes from ``config.json``; what a mixer needs is checked here, so that a folder with a missing
or mistyped key is refused before any weight is read.  Two sizes are given by a checkpoint's tensor shapes rather than by
a key (the rows of an attention layer's distance table, the inner width of a time-mixing layer's decay):
``with_tensor_shapes`` takes them from there; ``bias_rows`` / ``decay_rank`` in a mixer's object say them where there is
no checkpoint yet (random weights).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig, eos_ids, optional, require

MIXER_TYPES = ("lightning", "attention", "wkv")


def _section(raw: Dict[str, Any], key: str, where: str) -> Dict[str, Any]:
    value = raw.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {where}`{key}` must be an object")
    return value


def _positive(raw: Dict[str, Any], key: str, where: str) -> int:
    try:
        value = require(raw, key, int)
    except ConfigError as err:
        raise ConfigError(f"config.json: {where}: {err}") from None
    if value <= 0:
        raise ConfigError(f"config.json: {where}`{key}` must be positive, got {value}")
    return value


def _number(raw: Dict[str, Any], key: str, where: str) -> float:
    try:
        return require(raw, key, float)
    except ConfigError as err:
        raise ConfigError(f"config.json: {where}: {err}") from None


@dataclass
class LakulixLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]

    @classmethod
    def parse(cls, raw: Any, index: int) -> "LakulixLayer":
        where = f"layers[{index}]: "
        if not isinstance(raw, dict):
            raise ConfigError(f"config.json: {where}must be an object")
        kind = raw.get("type")
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {where}`type` {kind!r} is not one of {list(MIXER_TYPES)}")
        m = _section(raw, "mixer", where)
        mixer: Dict[str, Any] = {"heads": _positive(m, "heads", where), "dim": _positive(m, "dim", where)}
        if kind == "lightning":
            mixer["vdim"] = _positive(m, "vdim", where)
            decay = m.get("decay")
            if not isinstance(decay, list) or len(decay) != mixer["heads"] or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
                raise ConfigError(f"config.json: {where}`decay` must list one number per head")
            mixer["decay"] = [float(d) for d in decay]
        elif kind == "attention":
            mixer["vdim"] = _positive(m, "vdim", where)
            mixer["kv_heads"] = _positive(m, "kv_heads", where)
            if mixer["heads"] % mixer["kv_heads"] != 0:
                raise ConfigError(f"config.json: {where}{mixer['heads']} heads cannot share {mixer['kv_heads']} kv heads evenly")
            mixer["scale"] = _number(m, "scale", where)
            mixer["bias_max"] = _number(m, "bias_max", where)
            temp = _section(m, "q_temp", where)
            mixer["q_temp"] = {"coef": _number(temp, "coef", where), "every": _positive(temp, "every", where)}
            if m.get("bias_rows") is not None:          # optional: a checkpoint's distance table says it by its shape
                mixer["bias_rows"] = _positive(m, "bias_rows", where)
        elif m.get("decay_rank") is not None:           # optional: a checkpoint's decay matrices say it by their shape
            mixer["decay_rank"] = _positive(m, "decay_rank", where)
        mlp = raw.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict):
                raise ConfigError(f"config.json: {where}`mlp` must be an object or null")
            if mlp.get("kind") != "dense":
                raise ConfigError(f"config.json: {where}`mlp.kind` {mlp.get('kind')!r} is not supported (dense)")
            mlp = {"kind": "dense", "ff": _positive(mlp, "ff", where)}
        return cls(kind, mixer, mlp)

    def to_json_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": dict(self.mixer), "mlp": dict(self.mlp) if self.mlp is not None else None}


@dataclass
class LakulixConfig(ModelConfig):
    layers: List[LakulixLayer] = field(default_factory=list)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    norm_eps: float = 0.0
    logit_softcap: Optional[float] = None

    ARCHITECTURE = "Lakulix"
    MODEL_TYPE = "lakulix"

    @property
    def layer_runs(self) -> List[int]:
        """The order layers run in: those of the loop ``loop_times`` times in a row, the others once."""
        n = len(self.layers)
        return (list(range(self.loop_start)) + list(range(self.loop_start, self.loop_stop)) * self.loop_times
                + list(range(self.loop_stop, n)))

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], generation: Optional[Dict[str, Any]] = None) -> "LakulixConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: `layers` must be a non-empty list")
        layers = [LakulixLayer.parse(layer, i) for i, layer in enumerate(layers_raw)]
        start, stop, times = 0, 0, 1
        loop = raw.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError("config.json: `loop` must be an object")
            start, stop, times = require(loop, "start", int), require(loop, "stop", int), require(loop, "times", int)
            if not 0 <= start <= stop <= len(layers) or times < 1:
                raise ConfigError(f"config.json: `loop` {loop!r} does not fit {len(layers)} layers")
        norm = _section(raw, "norm", "")
        softcap = optional(raw, "logit_softcap", float)
        if softcap is not None and softcap <= 0:
            raise ConfigError(f"config.json: `logit_softcap` must be positive, got {softcap}")
        eos = eos_ids(raw.get("eos_token_id"))
        if generation is not None and generation.get("eos_token_id") is not None:
            eos = eos_ids(generation.get("eos_token_id"))
        return cls(architecture=cls.ARCHITECTURE, model_type=cls.MODEL_TYPE, vocab_size=_positive(raw, "vocab", ""),
                   hidden_size=_positive(raw, "width", ""), max_position_embeddings=_positive(raw, "max_positions", ""),
                   eos_token_ids=eos, raw=dict(raw), layers=layers, loop_start=start, loop_stop=stop, loop_times=times,
                   norm_eps=_number(norm, "eps", "norm: "), logit_softcap=softcap)

    def with_tensor_shapes(self, shapes: Dict[str, Any]) -> "LakulixConfig":
        """Takes the sizes that a checkpoint's tensors give by their shapes: ``l<i>.mix.rel`` is ``[bias_rows, heads]``,
        ``l<i>.mix.w1`` is ``[decay_rank, width]``."""
        for i, layer in enumerate(self.layers):
            if layer.type == "attention" and f"l{i}.mix.rel" in shapes and len(shapes[f"l{i}.mix.rel"]) == 2:
                layer.mixer["bias_rows"] = int(shapes[f"l{i}.mix.rel"][0])
            if layer.type == "wkv" and f"l{i}.mix.w1" in shapes and len(shapes[f"l{i}.mix.w1"]) == 2:
                layer.mixer["decay_rank"] = int(shapes[f"l{i}.mix.w1"][0])
        return self

    def to_json_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {
            "architecture": self.ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
            "max_positions": self.max_position_embeddings, "layers": [layer.to_json_dict() for layer in self.layers],
            "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times},
            "norm": {"eps": self.norm_eps},
        }
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
