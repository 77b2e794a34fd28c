"""Lakulix as data: pre-norm layers with a Dynamic Tanh norm whose mixers differ from layer to layer (linear attention
with a fixed decay, attention with sigmoid weights and a distance table, time mixing with a token-dependent decay), a
PolyNorm feed-forward where a layer has one, a learned position table beside the token table, a loop over a run of
layers, and a tanh cap on the logits.

Tensor names: ``embed``, ``pos``, ``l<i>.norm1`` (with ``.b`` and ``.alpha`` beside it), ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.  A layer of the loop runs several times with the same weights; every run is a schedule entry
of its own and so has a cache or state of its own.  Two sizes are not keys of ``config.json`` but shapes of the
checkpoint's tensors (``resolve_shapes``): the rows of ``l<i>.mix.rel`` and the inner width of ``l<i>.mix.w1``.
"""
from __future__ import annotations

from typing import Dict, Tuple

from ..config.lakulix import LakulixConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import register_architecture

#: the decay's inner width and the rows of a distance table where neither a checkpoint nor config.json says (random weights)
DEFAULT_DECAY_RANK = 32
DEFAULT_BIAS_ROWS = 32

NORM_NAMES = ("", "b", "alpha")       # the weight is the tensor `<name>` itself


def _mixer(cfg: LakulixConfig, index: int) -> PartSpec:
    layer = cfg.layers[index]
    m, h, eps = layer.mixer, cfg.hidden_size, cfg.norm_eps
    if layer.type == "lightning":
        return PartSpec("linear_attention", {"hidden": h, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                                             "decay": m["decay"], "norm_eps": eps})
    if layer.type == "attention":
        rows = m.get("bias_rows", DEFAULT_BIAS_ROWS)
        return PartSpec("sigmoid_attention", {
            "hidden": h, "heads": m["heads"], "kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
            "scale": m["scale"], "qk_norm": True, "norm_eps": eps, "temp_coef": m["q_temp"]["coef"],
            "temp_every": m["q_temp"]["every"], "bias_rows": rows, "bias_max": m["bias_max"], "head_bias": True,
            "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "rel": "rel", "pb": "pb"}})
    return PartSpec("wkv", {"hidden": h, "heads": m["heads"], "dim": m["dim"], "decay_rank": m.get("decay_rank", DEFAULT_DECAY_RANK),
                            "norm_eps": eps})


def resolve_shapes(cfg: LakulixConfig, shapes: Dict[str, Tuple[int, ...]]) -> LakulixConfig:
    """Sizes that only the checkpoint gives are taken from the shapes of its tensors, by name, before the model is built."""
    return cfg.with_tensor_shapes(shapes)


def build_spec(cfg: LakulixConfig) -> ModelSpec:
    h = cfg.hidden_size
    norm = PartSpec("dynamic_tanh", {"dim": h, "eps": cfg.norm_eps, "names": NORM_NAMES})
    layers = []
    for i, layer in enumerate(cfg.layers):
        ffn = None
        if layer.mlp is not None:
            ffn = PartSpec("polynorm_mlp", {"hidden": h, "intermediate": layer.mlp["ff"], "eps": cfg.norm_eps})
        layers.append(LayerSpec(block="prenorm", norm=norm, mixer=_mixer(cfg, i), feedforward=ffn, prefix=f"l{i}",
                                names={"norm1": "norm1", "mixer": "mix", "norm2": "norm2", "feedforward": "mlp"}))
    return ModelSpec(
        hidden_size=h,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_table", {"vocab": cfg.vocab_size, "hidden": h, "name": "embed", "tensor": "embed",
                                           "positions": cfg.max_position_embeddings, "position_tensor": "pos"}),
        final_norm=PartSpec("dynamic_tanh", {"dim": h, "eps": cfg.norm_eps, "name": "final.norm", "names": NORM_NAMES}),
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": h, "name": "head", "tensor": "head",
                                 "softcap": cfg.logit_softcap}),
        layers=layers,
        schedule=[ScheduleEntry(i) for i in cfg.layer_runs],
    )


register_architecture(LakulixConfig.ARCHITECTURE, LakulixConfig.MODEL_TYPE, LakulixConfig, build_spec, resolve_shapes)
