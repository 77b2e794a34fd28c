"""A plain, slow implementation of the Lakulix decoder: whole sequences, no cache, one function per
mechanism, torch on the CPU (float64 by default).  It shares no code with ``marin_b200``: it reads
``config.json`` with ``json`` and the weights with the ``safetensors`` library, and every recurrence is a
Python loop over the tokens.

Notation: ``x`` is the residual stream ``[T, width]``, ``h`` a mixer's (normed) input, ``p`` a position
counted from 0 in its sequence, ``W x`` a matrix stored ``[out, in]`` applied to a vector.
"""
from __future__ import annotations

import json
import math
import os
from typing import Callable, Dict, List, Optional, Sequence

import torch


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as fh:
        return json.load(fh)


def read_weights(model_dir: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    out = {}
    for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items():
        out[k] = v.to(dtype) if v.is_floating_point() else v
    return out


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return x @ w.t()


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def dynamic_tanh(x: torch.Tensor, alpha: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """tanh(alpha x) w + b, element by element: no statistic of the row enters."""
    return torch.tanh(alpha * x) * w + b


def embed(ids: Sequence[int], table: torch.Tensor, pos_table: torch.Tensor, first_position: int = 0) -> torch.Tensor:
    """table[id] + pos_table[p], the position vector added as it is."""
    ids = torch.as_tensor(list(ids), dtype=torch.long)
    p = torch.arange(first_position, first_position + len(ids))
    return table[ids] + pos_table[p]


def lightning(h, w, prefix, heads, dim, vdim, decay, eps):
    """Linear attention with a fixed decay per head.  q = silu(W_q h), k = silu(W_k h), v = silu(W_v h);
    S_t = decay_h S_(t-1) + k_t v_t^T (S: dim x vdim, zero at the start); o_t = S_t^T q_t.  The heads side by side are
    divided by their common root mean square, times the weight, times sigmoid(W_g h), then W_o."""
    T = h.shape[0]
    q = silu(linear(h, w[prefix + ".q"])).view(T, heads, dim)
    k = silu(linear(h, w[prefix + ".k"])).view(T, heads, dim)
    v = silu(linear(h, w[prefix + ".v"])).view(T, heads, vdim)
    o = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for a in range(heads):
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        for t in range(T):
            S = float(decay[a]) * S + torch.outer(k[t, a], v[t, a])
            o[t, a] = S.t() @ q[t, a]
    o = unit_rms(o.reshape(T, heads * vdim), eps) * w[prefix + ".norm"]
    return linear(o * sigmoid(linear(h, w[prefix + ".g"])), w[prefix + ".o"])


def distance_bucket(n: int, rows: int, farthest: float) -> int:
    """Row of the distance table for distance n >= 0: the first half of the rows one distance each, the other half
    spread evenly over the logarithm of the distance up to ``farthest``; the last row takes everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(farthest / half) * (rows - half))))


def sigmoid_attention(h, w, prefix, heads, kv_heads, dim, vdim, scale, farthest, temp_coef, temp_every, eps):
    """Causal attention without a softmax.  q and k get a per-head RMS norm (weight shared by the heads), q is
    multiplied by 1 + coef ln(floor((p + 1) / every) + 1); score = q.k scale + rel[bucket(i - j), head]; the weight
    of key j <= i is sigmoid(score + pb[head]), and weights are not normalised over the keys."""
    T = h.shape[0]
    q = linear(h, w[prefix + ".q"]).view(T, heads, dim)
    k = linear(h, w[prefix + ".k"]).view(T, kv_heads, dim)
    v = linear(h, w[prefix + ".v"]).view(T, kv_heads, vdim)
    q = unit_rms(q, eps) * w[prefix + ".q.norm"]
    k = unit_rms(k, eps) * w[prefix + ".k.norm"]
    rel, pb = w[prefix + ".rel"], w[prefix + ".pb"]
    rows = rel.shape[0]
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    group = heads // kv_heads
    for i in range(T):
        temp = 1.0 + temp_coef * math.log((i + 1) // temp_every + 1)
        for a in range(heads):
            g = a // group
            qi = q[i, a] * temp
            acc = torch.zeros(vdim, dtype=h.dtype)
            for j in range(i + 1):
                s = float(qi @ k[j, g]) * scale + float(rel[distance_bucket(i - j, rows, farthest), a])
                acc = acc + (1.0 / (1.0 + math.exp(-(s + float(pb[a]))))) * v[j, g]
            out[i, a] = acc
    return linear(out.reshape(T, heads * vdim), w[prefix + ".o"])


def sigmoid_attention_fast(h, w, prefix, heads, kv_heads, dim, vdim, scale, farthest, temp_coef, temp_every, eps):
    """The same as ``sigmoid_attention`` with the loops over keys written as matrix operations (for long sequences)."""
    T = h.shape[0]
    q = unit_rms(linear(h, w[prefix + ".q"]).view(T, heads, dim), eps) * w[prefix + ".q.norm"]
    k = unit_rms(linear(h, w[prefix + ".k"]).view(T, kv_heads, dim), eps) * w[prefix + ".k.norm"]
    v = linear(h, w[prefix + ".v"]).view(T, kv_heads, vdim)
    temp = torch.tensor([1.0 + temp_coef * math.log((i + 1) // temp_every + 1) for i in range(T)], dtype=h.dtype)
    q = q * temp[:, None, None]
    rel, pb = w[prefix + ".rel"], w[prefix + ".pb"]
    rows = rel.shape[0]
    buckets = torch.tensor([distance_bucket(n, rows, farthest) for n in range(T)], dtype=torch.long)
    i = torch.arange(T)
    dist = (i[:, None] - i[None, :]).clamp(min=0)
    seen = i[:, None] >= i[None, :]
    group = heads // kv_heads
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for a in range(heads):
        g = a // group
        s = (q[:, a] @ k[:, g].t()) * scale + rel[:, a][buckets[dist]] + pb[a]
        wgt = torch.where(seen, sigmoid(s), torch.zeros((), dtype=h.dtype))
        out[:, a] = wgt @ v[:, g]
    return linear(out.reshape(T, heads * vdim), w[prefix + ".o"])


def wkv(h, w, prefix, heads, dim, eps):
    """Time mixing with a data-dependent decay.  With h' the row before (zeros before the first): each of r, k, v,
    g, w reads h + (h' - h) mu_s.  decay_t = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0)) per head and key channel.
    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t; then S_t = diag(decay_t) S_(t-1) + k_t v_t^T.  Each head's o is divided
    by its root mean square; heads side by side, times the weight, times silu(W_g mix_g), then W_o."""
    T = h.shape[0]
    before = torch.cat([torch.zeros(1, h.shape[1], dtype=h.dtype), h[:-1]], dim=0)

    def mix(s):
        return h + (before - h) * w[prefix + ".mu." + s]

    r = linear(mix("r"), w[prefix + ".r"]).view(T, heads, dim)
    k = linear(mix("k"), w[prefix + ".k"]).view(T, heads, dim)
    v = linear(mix("v"), w[prefix + ".v"]).view(T, heads, dim)
    gate = silu(linear(mix("g"), w[prefix + ".g"]))
    decay = torch.exp(-torch.exp(linear(torch.tanh(linear(mix("w"), w[prefix + ".w1"])), w[prefix + ".w2"]) + w[prefix + ".w0"]))
    decay = decay.view(T, heads, dim)
    u = w[prefix + ".u"]
    o = torch.zeros(T, heads, dim, dtype=h.dtype)
    for a in range(heads):
        S = torch.zeros(dim, dim, dtype=h.dtype)
        for t in range(T):
            kv = torch.outer(k[t, a], v[t, a])
            o[t, a] = (S + u[a][:, None] * kv).t() @ r[t, a]
            S = decay[t, a][:, None] * S + kv
    o = unit_rms(o, eps).reshape(T, heads * dim) * w[prefix + ".norm"]
    return linear(o * gate, w[prefix + ".o"])


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    """a N(z) + b N(z^2) + c N(z^3) + e, powers element by element, N = a row divided by its root mean square."""
    a, b, c, e = (coef[i] for i in range(4))
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def dense_mlp(h, w, prefix, eps):
    return linear(polynorm(linear(h, w[prefix + ".up"]), w[prefix + ".act"], eps), w[prefix + ".down"])


def layer_runs(cfg: dict) -> List[int]:
    """The order layers run in: those of the loop ``times`` times in a row, the others once."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    order = list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + list(range(loop["stop"], n))
    return order


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int], observe: Optional[Callable] = None,
            fast: bool = True) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``observe(run, x)`` gets the residual stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = embed(ids, w["embed"], w["pos"])

    def norm(name, t):
        return dynamic_tanh(t, w[name + ".alpha"], w[name], w[name + ".b"])

    for run, i in enumerate(layer_runs(cfg)):
        layer, name = cfg["layers"][i], f"l{i}"
        m = layer["mixer"]
        h = norm(name + ".norm1", x)
        if layer["type"] == "lightning":
            y = lightning(h, w, name + ".mix", m["heads"], m["dim"], m["vdim"], m["decay"], eps)
        elif layer["type"] == "attention":
            fn = sigmoid_attention_fast if fast else sigmoid_attention
            y = fn(h, w, name + ".mix", m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], m["bias_max"],
                   m["q_temp"]["coef"], m["q_temp"]["every"], eps)
        elif layer["type"] == "wkv":
            y = wkv(h, w, name + ".mix", m["heads"], m["dim"], eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']}")
        x = x + y
        if layer.get("mlp") is not None:
            x = x + dense_mlp(norm(name + ".norm2", x), w, name + ".mlp", eps)
        if observe is not None:
            observe(run, x)
    logits = linear(norm("final.norm", x), w["head"])
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
