"""Fegarax as data: pre-norm layers over several copies of the residual stream (hyper-connections), each with a
grouped-query softmax attention (biases, an RMS norm over the whole of q and of k, partly rotated heads with rescaled
frequencies, a chunked mask, a sink in the softmax, values mixed with the first such layer's, a sigmoid output gate) and a
routed feed-forward (sigmoid scores, the chosen experts' inputs scaled by them).  The embedding is scaled, the head is the
unscaled table.

Tensor names: ``embed``, ``l<i>.norm1`` / ``norm2`` (weights around zero), ``l<i>.mix.{q,k,v}`` with ``.b`` beside them,
``l<i>.mix.{q,k}.norm``, ``l<i>.mix.vmix``, ``l<i>.mix.g``, ``l<i>.mix.o``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.{gate,up,down}``,
``l<i>.hc<q>.{in,out,mix}``, ``final.norm``.
"""
from __future__ import annotations

from ..config.fegarax import FegaraxConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import register_architecture

MIXER_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
               "q_norm": "q.norm", "k_norm": "k.norm", "lam": "vmix"}
EXPERT_NAMES = {"router": "router", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down"}


def _position(m: dict) -> PartSpec:
    rot = m["rot"]
    if rot is None:
        return PartSpec("none", {})
    params = {"head_dim": m["dim"], "theta": rot["base"], "rotary_dim": rot["dims"]}
    if rot["scaling"] is None:
        return PartSpec("rope", params)
    return PartSpec("rope_yarn", dict(params, **rot["scaling"]))


def build_spec(cfg: FegaraxConfig) -> ModelSpec:
    h = cfg.hidden_size
    norm = PartSpec("rmsnorm", {"dim": h, "eps": cfg.norm_eps, "unit_offset": True, "tensor": ""})
    layers = []
    seen_value_mix = False
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        mixer = PartSpec("sink_attention", {
            "hidden": h, "heads": m["heads"], "kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
            "scale": m["scale"], "bias": True, "qk_norm": "whole", "norm_eps": cfg.norm_eps, "position": _position(m),
            "chunk": m["mask"]["size"] if m["mask"] is not None else None, "sink": True,
            "value_mix": "v" if m["v_mix"] else None, "first_of_mix": m["v_mix"] and not seen_value_mix, "gate": True,
            "names": MIXER_NAMES})
        seen_value_mix = seen_value_mix or m["v_mix"]
        ffn = None
        if layer.mlp is not None:
            ffn = PartSpec("routed_experts", {"hidden": h, "intermediate": layer.mlp["expert"]["ff"], "experts": layer.mlp["router"]["experts"],
                                              "top": layer.mlp["router"]["top"], "score": "sigmoid", "renormalize": False,
                                              "weight_on": "input", "names": EXPERT_NAMES})
        names = {"norm1": "norm1", "mixer": "mix", "norm2": "norm2", "feedforward": "mlp"}
        if cfg.streams is None:
            layers.append(LayerSpec(block="prenorm", norm=norm, mixer=mixer, feedforward=ffn, prefix=f"l{i}", names=names))
        else:
            layers.append(LayerSpec(block="hyper_prenorm", norm=norm, mixer=mixer, feedforward=ffn, prefix=f"l{i}", names=names,
                                    block_params={"streams": cfg.streams}))
    return ModelSpec(
        hidden_size=h,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_table", {"vocab": cfg.vocab_size, "hidden": h, "name": "embed", "tensor": "embed",
                                           "scale": cfg.embedding_scale}),
        final_norm=PartSpec("rmsnorm", {"dim": h, "eps": cfg.norm_eps, "name": "final.norm", "unit_offset": True, "tensor": ""}),
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": h, "name": "head", "tied": True}),
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(len(cfg.layers))],
        streams=cfg.streams if cfg.streams is not None else 0,
        # a layer outside the value mixing has no use for a mixing number, should a checkpoint bring one
        ignorable=tuple(f"l{i}.mix.vmix" for i, layer in enumerate(cfg.layers) if not layer.mixer["v_mix"]),
    )


register_architecture(FegaraxConfig.ARCHITECTURE, FegaraxConfig.MODEL_TYPE, FegaraxConfig, build_spec)
