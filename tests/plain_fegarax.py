"""A plain, slow Fegarax in float64: one function per mechanism, loops where a loop says it best.

It shares nothing with the package: tensors come as a dict of torch tensors (any dtype; everything is widened to
float64), the configuration as the raw dict of ``config.json``.  A whole sequence is computed at once, token by token
where the mechanism is causal, with no cache: what the engine gives for any cut of the prompt, any batch and any page
must equal this up to rounding.

Notation: ``x`` a residual stream ``[T, width]``, ``h`` a sublayer's normed input, ``p`` a position, matrices ``[out, in]``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def f64(t) -> torch.Tensor:
    return t.to(F64)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, one_plus: bool) -> torch.Tensor:
    """Rows over their root mean square (eps under the root), times ``w`` or ``1 + w``."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y * ((1.0 + f64(w)) if one_plus else f64(w))


def rotary_frequencies(rot: dict):
    """Per pair ``i < dims/2`` the angle per position, and the factor on cos and sin.  Without ``scaling``: ``base^(-2i/dims)``
    and 1.  With it, frequencies below the ramp are kept, those above are divided by ``factor``, in between blended."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F64), 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def dim_of(turns: float) -> float:
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """``x`` ``[T, heads, dim]``: the first ``dims`` of every head are rotated in pairs ``(i, i + dims/2)``."""
    if not rot:
        return x
    freq, mag = rotary_frequencies(rot)
    dims = int(rot["dims"])
    half = dims // 2
    ang = positions.to(F64)[:, None] * freq[None, :]             # [T, half]
    cos, sin = torch.cos(ang)[:, None, :] * mag, torch.sin(ang)[:, None, :] * mag
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def visible(T: int, mask: Optional[dict]) -> torch.Tensor:
    """``[T, T]`` booleans: whether position ``i`` (row) looks at position ``j`` (column): never ahead; with a chunked mask only
    inside its own chunk, chunks counted from position 0."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    see = j <= i
    if mask and mask.get("size"):
        size = int(mask["size"])
        see = see & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))
    return see


def sink_softmax_mix(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, mask: Optional[dict], sink: bool = True) -> torch.Tensor:
    """One head.  ``q`` ``[T, d]``, ``k`` ``[T, d]``, ``v`` ``[T, dv]``.  Weights ``exp(s_j) / (1 + sum_j exp(s_j))`` over the keys a
    position sees: the one stands for a key of score 0 that has no value (``sink=False``: an ordinary softmax)."""
    s = (q @ k.T) * scale
    s = s.masked_fill(~visible(q.shape[0], mask), -math.inf)
    m = s.max(dim=-1, keepdim=True).values
    if sink:
        m = torch.clamp(m, min=0.0)
    e = torch.exp(s - m)
    return (e @ v) / ((torch.exp(-m) if sink else 0.0) + e.sum(dim=-1, keepdim=True))


def attention_mixer(h: torch.Tensor, positions: torch.Tensor, W: Dict[str, torch.Tensor], pre: str, m: dict, eps: float,
                    shared: dict, first_vmix: bool, sink: bool = True) -> torch.Tensor:
    """The attention mixer over a whole sequence.  ``shared['v_first']`` carries the values of the first value-mixing layer."""
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = h @ f64(W[pre + "q"]).T + f64(W[pre + "q.b"])
    k = h @ f64(W[pre + "k"]).T + f64(W[pre + "k.b"])
    v = h @ f64(W[pre + "v"]).T + f64(W[pre + "v.b"])
    q = rms_norm(q, W[pre + "q.norm"], eps, False)                 # over all heads at once
    k = rms_norm(k, W[pre + "k.norm"], eps, False)
    q = rotate(q.view(T, H, d), positions, m.get("rot"))
    k = rotate(k.view(T, G, d), positions, m.get("rot"))
    if m.get("v_mix"):
        if first_vmix:
            shared["v_first"] = v
        else:
            lam = float(f64(W[pre + "vmix"]))
            v = (1.0 - lam) * v + lam * shared["v_first"]
    v = v.view(T, G, dv)
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        heads.append(sink_softmax_mix(q[:, hh], k[:, g], v[:, g], float(m["scale"]), m.get("mask"), sink))
    o = torch.cat(heads, dim=-1)
    o = o * torch.sigmoid(h @ f64(W[pre + "g"]).T)
    return o @ f64(W[pre + "o"]).T


def router_margins(h: torch.Tensor, W: Dict[str, torch.Tensor], pre: str, mlp: dict) -> torch.Tensor:
    """Per token, how far the last chosen expert's router logit lies above the best one left out (inf if none is left out)."""
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = (h @ f64(W[pre + "router"]).T).sort(dim=-1, descending=True).values
    return z[:, top - 1] - z[:, top] if top < E else torch.full((h.shape[0],), math.inf, dtype=F64)


def routed_experts(h: torch.Tensor, W: Dict[str, torch.Tensor], pre: str, mlp: dict, score: str = "sigmoid", renormalize: bool = False,
                   weight_on: str = "input") -> torch.Tensor:
    """Sigmoid scores, the ``top`` largest chosen, each chosen expert fed ``score * h``; outputs summed.  (The other settings
    of the part: scores from a softmax over all experts, weights renormalised over the chosen ones, the weight on the output.)"""
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = h @ f64(W[pre + "router"]).T
    s = torch.sigmoid(z) if score == "sigmoid" else torch.softmax(z, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(z[t, e]), e))[:top]
        total = sum(float(s[t, e]) for e in order) if renormalize else 1.0
        for e in order:
            w = s[t, e] / total
            x = w * h[t] if weight_on == "input" else h[t]
            gate = f64(W[f"{pre}e{e}.gate"]) @ x
            up = f64(W[f"{pre}e{e}.up"]) @ x
            y = f64(W[f"{pre}e{e}.down"]) @ (gate * torch.sigmoid(gate) * up)
            out[t] += y if weight_on == "input" else w * y
    return out


def hyper_step(streams: List[torch.Tensor], w_in, w_out, w_mix, fn):
    """One sublayer over the streams: ``u = sum_s in[s] x_s``, ``y = fn(u)``, ``x_t <- sum_s mix[s, t] x_s + out[t] y``."""
    n = len(streams)
    u = sum(w_in[s] * streams[s] for s in range(n))
    y = fn(u)
    return [sum(w_mix[s, t] * streams[s] for s in range(n)) + w_out[t] * y for t in range(n)]


def read_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    import os

    return load_file(os.path.join(model_dir, "model.safetensors"))


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], margins: Optional[list] = None):
    """Logits ``[T, vocab]`` and the residual stream after every layer ``[layers, T, width]`` (the sum of the streams).
    ``margins`` collects every routed layer's ``router_margins``."""
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    positions = torch.arange(T)
    x0 = f64(W["embed"])[torch.tensor(tokens)] * float(cfg.get("embedding", {}).get("scale", 1.0))
    S = cfg.get("streams")
    streams = [x0.clone() for _ in range(int(S))] if S else [x0.clone()]
    shared: dict = {}
    seen_vmix = False
    after = []
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."

        def mixer(hh):
            nonlocal seen_vmix
            first = bool(layer["mixer"].get("v_mix")) and not seen_vmix
            y = attention_mixer(hh, positions, W, pre + "mix.", layer["mixer"], eps, shared, first)
            if layer["mixer"].get("v_mix"):
                seen_vmix = True
            return y

        subs = [(1, mixer)]
        def experts(hh):
            if margins is not None:
                margins.append(router_margins(hh, W, pre + "mlp.", layer["mlp"]))
            return routed_experts(hh, W, pre + "mlp.", layer["mlp"])

        if layer.get("mlp") is not None:
            subs.append((2, experts))
        for qn, fn in subs:
            if S:
                streams = hyper_step(streams, f64(W[f"{pre}hc{qn}.in"]), f64(W[f"{pre}hc{qn}.out"]), f64(W[f"{pre}hc{qn}.mix"]),
                                     lambda u: fn(rms_norm(u, W[f"{pre}norm{qn}"], eps, True)))
            else:
                streams[0] = streams[0] + fn(rms_norm(streams[0], W[f"{pre}norm{qn}"], eps, True))
        after.append(sum(streams))
    x = sum(streams)
    logits = rms_norm(x, W["final.norm"], eps, True) @ f64(W["embed"]).T
    return logits, torch.stack(after)
