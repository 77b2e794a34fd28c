"""Small Lakulix configurations and random weights for the tests, written with the ``safetensors`` library (not with the
engine's own writer).  Weights are drawn so that every mechanism matters: mixing coefficients spread over (0, 1), decays
from fast to slow, distance tables and head offsets of order one, activation coefficients all non-zero.  Values are
rounded to bfloat16 so that a 32-bit engine and the plain implementation read the same numbers.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict

import torch

# Layers of three kinds in an order of their own, a loop that starts after the first layer and runs three times, value heads
# wider than key heads, two kv heads, an even distance table that saturates inside the test's lengths, a temperature
# that changes every 16 positions.
CONFIG_A = {
    "architecture": "Lakulix", "vocab": 97, "width": 64, "max_positions": 160, "norm": {"eps": 1e-5}, "logit_softcap": 8.0,
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 80},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "bias_max": 40, "q_temp": {"coef": 0.4, "every": 16}}},
        {"type": "lightning", "mlp": None, "mixer": {"heads": 3, "dim": 8, "vdim": 16, "decay": [0.5, 0.9, 0.995]}},
        {"type": "wkv", "mlp": {"kind": "dense", "ff": 48}, "mixer": {"heads": 2, "dim": 16}},
    ],
}
SHAPES_A = {"rows": 10, "rank": 8}
# No loop and no cap on the logits; an odd distance table with a fractional reach; value heads narrower than key heads and
# as many kv heads as heads; a linear-attention head whose values span more than one block of columns; an inner decay
# width that is no multiple of 8; sizes that are no powers of two.
CONFIG_B = {
    "architecture": "Lakulix", "vocab": 130, "width": 96, "max_positions": 200, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "wkv", "mlp": None, "mixer": {"heads": 3, "dim": 24}},
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.2, "bias_max": 25.5, "q_temp": {"coef": 0.25, "every": 7}}},
        {"type": "lightning", "mlp": {"kind": "dense", "ff": 136}, "mixer": {"heads": 2, "dim": 40, "vdim": 72, "decay": [0.8, 0.97]}},
    ],
}
SHAPES_B = {"rows": 7, "rank": 12}
# One layer of each kind looped twice from the start to the end, heads of 64 and 128 (the sizes tensor-core kernels are made for).
CONFIG_C = {
    "architecture": "Lakulix", "vocab": 160, "width": 256, "max_positions": 320, "norm": {"eps": 1e-6}, "logit_softcap": 20.0,
    "loop": {"start": 0, "stop": 3, "times": 2},
    "layers": [
        {"type": "lightning", "mlp": None, "mixer": {"heads": 2, "dim": 64, "vdim": 128, "decay": [0.9, 0.999]}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 512},
         "mixer": {"heads": 8, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.11, "bias_max": 100, "q_temp": {"coef": 0.2, "every": 48}}},
        {"type": "wkv", "mlp": None, "mixer": {"heads": 4, "dim": 64}},
    ],
}
SHAPES_C = {"rows": 12, "rank": 24}
CONFIGS = {"A": (CONFIG_A, SHAPES_A), "B": (CONFIG_B, SHAPES_B), "C": (CONFIG_C, SHAPES_C)}
PAGE = {"A": 4, "B": 8, "C": 16}


def random_weights(raw: dict, shapes: dict, seed: int) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    width, vocab = raw["width"], raw["vocab"]

    def normal(*shape, std=1.0, mean=0.0):
        return torch.randn(shape, generator=g) * std + mean

    def matrix(rows, cols, gain=1.0):
        return normal(rows, cols, std=gain / math.sqrt(cols))

    def uniform(*shape, lo=0.0, hi=1.0):
        return torch.rand(shape, generator=g) * (hi - lo) + lo

    w: Dict[str, torch.Tensor] = {"embed": normal(vocab, width), "pos": normal(raw["max_positions"], width, std=0.5),
                                  "head": matrix(vocab, width, 2.0)}

    def norm(name):
        w[name] = normal(width, std=0.2, mean=1.0)
        w[name + ".b"] = normal(width, std=0.2)
        w[name + ".alpha"] = uniform(lo=0.4, hi=1.2).reshape(())

    norm("final.norm")
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}", layer["mixer"]
        norm(p + ".norm1")
        H, d = m["heads"], m["dim"]
        if layer["type"] == "lightning":
            dv = m["vdim"]
            w[p + ".mix.q"], w[p + ".mix.k"] = matrix(H * d, width, 2.0), matrix(H * d, width, 2.0)
            w[p + ".mix.v"], w[p + ".mix.g"] = matrix(H * dv, width, 2.0), matrix(H * dv, width, 2.0)
            w[p + ".mix.o"] = matrix(width, H * dv)
            w[p + ".mix.norm"] = normal(H * dv, std=0.2, mean=1.0)
        elif layer["type"] == "attention":
            G, dv = m["kv_heads"], m["vdim"]
            w[p + ".mix.q"], w[p + ".mix.k"], w[p + ".mix.v"] = matrix(H * d, width), matrix(G * d, width), matrix(G * dv, width)
            w[p + ".mix.q.norm"], w[p + ".mix.k.norm"] = normal(d, std=0.3, mean=1.5), normal(d, std=0.3, mean=1.5)
            w[p + ".mix.rel"] = normal(shapes["rows"], H, std=1.5)
            w[p + ".mix.pb"] = normal(H, std=0.5, mean=-2.0)
            w[p + ".mix.o"] = matrix(width, H * dv, 0.5)
        else:
            n = H * d
            for s in "rkvgw":
                w[f"{p}.mix.mu.{s}"] = uniform(width)
            for s in "rkvg":
                w[f"{p}.mix.{s}"] = matrix(n, width)
            w[p + ".mix.w1"] = matrix(shapes["rank"], width)
            w[p + ".mix.w2"] = matrix(n, shapes["rank"], 2.0)
            w[p + ".mix.w0"] = uniform(n, lo=-4.0, hi=0.5)       # decays from exp(-exp(-4)) = 0.98 down to 0.19
            w[p + ".mix.u"] = normal(H, d, std=0.5)
            w[p + ".mix.norm"] = normal(n, std=0.2, mean=1.0)
            w[p + ".mix.o"] = matrix(width, n)
        if layer.get("mlp") is not None:
            norm(p + ".norm2")
            ff = layer["mlp"]["ff"]
            w[p + ".mlp.up"], w[p + ".mlp.down"] = matrix(ff, width), matrix(width, ff, 0.7)
            w[p + ".mlp.act"] = torch.tensor([0.8, -0.5, 0.3, 0.1]) + normal(4, std=0.05)
    return {k: v.to(torch.bfloat16) for k, v in w.items()}


def write_model(path: str, raw: dict, weights: Dict[str, torch.Tensor]) -> str:
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(raw, fh)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(path, "model.safetensors"))
    return path


def make_model_dir(path: str, name: str, seed: int = 3) -> str:
    raw, shapes = CONFIGS[name]
    return write_model(path, raw, random_weights(raw, shapes, seed))
