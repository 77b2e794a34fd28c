"""Small Fegarax configurations and random weights for the tests, written with the ``safetensors`` library (not with the
engine's own writer).  Weights are drawn so that every mechanism matters: stream coefficients well away from the identity,
norm weights spread around zero, biases of order one, mixing numbers inside (0, 1), router logits spread over several
units.  Values are rounded to bfloat16 so that a 32-bit engine and the plain implementation read the same numbers.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict

import torch


def _attn(heads, kv, dim, vdim, scale, mask=None, rot=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if mask:
        m["mask"] = {"size": mask}
    if rot:
        m["rot"] = rot
    if v_mix:
        m["v_mix"] = True
    return m


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


YARN_A = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}
# Two streams; layers that differ in everything: a first layer outside the value mixing, chunks of 13 and of 5 positions and a
# layer without a mask, rotations of 8 of 16 dimensions with rescaled frequencies, of all dimensions without, and none at all;
# two, three and all of the experts chosen; a layer without feed-forward.
CONFIG_A = {
    "architecture": "Fegarax", "vocab": 97, "width": 64, "streams": 2, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _attn(4, 2, 16, 24, 0.3, mask=13, rot={"base": 100.0, "dims": 8, "scaling": YARN_A}), "mlp": _moe(40, 5, 2)},
        {"type": "attention", "mixer": _attn(2, 1, 24, 40, 0.25, mask=5, rot={"base": 50.0, "dims": 24}, v_mix=True), "mlp": None},
        {"type": "attention", "mixer": _attn(4, 1, 16, 40, 0.4, v_mix=True), "mlp": _moe(24, 3, 3)},
        {"type": "attention", "mixer": _attn(1, 1, 32, 40, 0.2, mask=64, rot={"base": 1000.0, "dims": 2}, v_mix=True), "mlp": _moe(16, 7, 3)},
    ],
}
# One plain residual stream (no `streams` key, no stream tensors), no embedding scale, as many kv heads as heads, a chunk of
# one position (every token sees itself and the sink only) beside a long one, frequencies whose ramp ends before it begins.
CONFIG_B = {
    "architecture": "Fegarax", "vocab": 130, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _attn(3, 3, 32, 16, 0.2, mask=1, rot={"base": 10000.0, "dims": 32, "scaling": {"factor": 2.0, "original": 4096, "fast": 1.0, "slow": 1.0}}, v_mix=True), "mlp": _moe(48, 4, 1)},
        {"type": "attention", "mixer": _attn(3, 3, 32, 16, 0.2, mask=100, rot={"base": 10000.0, "dims": 16, "scaling": {"factor": 16.0, "original": 64, "fast": 4.0, "slow": 2.0}}, v_mix=True), "mlp": _moe(48, 4, 2)},
    ],
}
# Four streams, heads of 64 and 128 (the sizes tensor-core kernels are made for) in groups of 4 and 2, chunks of exactly one
# key block and of a length that is no multiple of anything, eight experts of which two are chosen.
YARN_C = {"factor": 8.0, "original": 128, "fast": 16.0, "slow": 2.0}
CONFIG_C = {
    "architecture": "Fegarax", "vocab": 160, "width": 256, "streams": 4, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _attn(8, 2, 64, 64, 0.125, mask=64, rot={"base": 5000.0, "dims": 32, "scaling": YARN_C}, v_mix=True), "mlp": _moe(128, 8, 2)},
        {"type": "attention", "mixer": _attn(4, 2, 128, 64, 0.09, mask=150, rot={"base": 5000.0, "dims": 64, "scaling": YARN_C}, v_mix=True), "mlp": _moe(64, 8, 2)},
        {"type": "attention", "mixer": _attn(2, 2, 64, 64, 0.125, rot={"base": 5000.0, "dims": 64}, v_mix=True), "mlp": None},
    ],
}
# One stream kept as hyper-connections (the stream tensors exist, with one entry each).
CONFIG_D = {
    "architecture": "Fegarax", "vocab": 61, "width": 48, "streams": 1, "embedding": {"scale": 0.5}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _attn(2, 2, 16, 16, 0.25, mask=9, rot={"base": 100.0, "dims": 16}), "mlp": _moe(32, 6, 2)},
        {"type": "attention", "mixer": _attn(6, 2, 8, 16, 0.35, mask=30), "mlp": _moe(32, 2, 1)},
    ],
}
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D}
PAGE = {"A": 4, "B": 8, "C": 16, "D": 2}


def random_weights(raw: dict, seed: int) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    width, vocab = raw["width"], raw["vocab"]

    def normal(*shape, std=1.0, mean=0.0):
        return torch.randn(shape, generator=g) * std + mean

    def matrix(rows, cols, gain=1.0):
        return normal(rows, cols, std=gain / math.sqrt(cols))

    def uniform(*shape, lo=0.0, hi=1.0):
        return torch.rand(shape, generator=g) * (hi - lo) + lo

    w: Dict[str, torch.Tensor] = {"embed": normal(vocab, width, std=1.0 / float(raw.get("embedding", {}).get("scale", 1.0))),
                                  "final.norm": normal(width, std=0.2)}
    S = raw.get("streams")
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}", layer["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        w[p + ".norm1"] = normal(width, std=0.2)
        w[p + ".mix.q"], w[p + ".mix.k"], w[p + ".mix.v"] = matrix(H * d, width), matrix(G * d, width), matrix(G * dv, width)
        w[p + ".mix.q.b"], w[p + ".mix.k.b"], w[p + ".mix.v.b"] = normal(H * d, std=0.5), normal(G * d, std=0.5), normal(G * dv, std=0.3)
        w[p + ".mix.q.norm"], w[p + ".mix.k.norm"] = normal(H * d, std=0.3, mean=1.5), normal(G * d, std=0.3, mean=1.5)
        if m.get("v_mix"):
            w[p + ".mix.vmix"] = uniform(lo=0.25, hi=0.75).reshape(())
        w[p + ".mix.g"] = matrix(H * dv, width, 2.0)
        w[p + ".mix.o"] = matrix(width, H * dv, 1.5)
        subs = ["hc1"]
        if layer.get("mlp") is not None:
            w[p + ".norm2"] = normal(width, std=0.2)
            ff, E = layer["mlp"]["expert"]["ff"], layer["mlp"]["router"]["experts"]
            w[p + ".mlp.router"] = matrix(E, width, 3.0)
            for e in range(E):
                w[f"{p}.mlp.e{e}.gate"], w[f"{p}.mlp.e{e}.up"] = matrix(ff, width, 2.0), matrix(ff, width, 2.0)
                w[f"{p}.mlp.e{e}.down"] = matrix(width, ff, 1.5)
            subs.append("hc2")
        if S:
            for hc in subs:
                w[f"{p}.{hc}.in"] = normal(S, std=0.3, mean=1.0 / S)
                w[f"{p}.{hc}.out"] = normal(S, std=0.3, mean=0.8)
                w[f"{p}.{hc}.mix"] = torch.eye(S) * 0.8 + normal(S, S, std=0.25)
    return {k: v.to(torch.bfloat16) for k, v in w.items()}


def write_model(path: str, raw: dict, weights: Dict[str, torch.Tensor]) -> str:
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(raw, fh)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(path, "model.safetensors"))
    return path


def make_model_dir(path: str, name: str, seed: int = 3) -> str:
    return write_model(path, CONFIGS[name], random_weights(CONFIGS[name], seed))
