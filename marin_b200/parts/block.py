"""How a layer's parts are arranged around the residual stream."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import Part, Runtime, spec_bytes
from .registry import lookup, register_block
from .spec import LayerSpec, TensorSpec


@register_block("prenorm")
class PreNormBlock(Part):
    """``h += mixer(norm1(h)); h += feedforward(norm2(h))`` — the residual stream ``h`` stays
    float32 and both parts add into it (crates/model/src/qwen3/layer.rs:56-103).  A layer whose spec has no
    feed-forward has the first sublayer only (and no second norm)."""

    def __init__(self, spec: LayerSpec):
        names = spec.names
        norm_cls = lookup("norm", spec.norm.kind)
        self.norm1 = norm_cls(name=f"{spec.prefix}.{names['norm1']}", **spec.norm.params)
        self.mixer = lookup("mixer", spec.mixer.kind)(name=f"{spec.prefix}.{names['mixer']}", **spec.mixer.params)
        self.norm2 = self.feedforward = None
        if spec.feedforward is not None:
            self.norm2 = norm_cls(name=f"{spec.prefix}.{names['norm2']}", **spec.norm.params)
            self.feedforward = lookup("feedforward", spec.feedforward.kind)(
                name=f"{spec.prefix}.{names['feedforward']}", **spec.feedforward.params)

    def parts(self) -> List[Part]:
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feedforward) if p is not None]

    def tensor_specs(self) -> List[TensorSpec]:
        return [s for p in self.parts() for s in p.tensor_specs()]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        for p in self.parts():
            p.load(tensors, rt)
        self.rt = rt

    def weight_bytes(self, dtype) -> int:
        return sum(p.weight_bytes(dtype) for p in self.parts())

    def bytes_read(self, tokens: int, dtype) -> int:
        return sum(p.bytes_read(tokens, dtype) for p in self.parts())

    def flops(self, tokens: int, pairs: int = 0) -> float:
        return sum(p.flops(tokens, pairs) for p in self.parts())

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        jobs: Dict[str, tuple] = {}
        for p in self.parts():
            jobs.update(p.kernel_jobs(dtype))
        return jobs

    #: ``forward`` takes ``x_in`` / ``next_block`` and returns the next block's input (see there)
    chains_norm = True

    def _rider(self, norm, producer, consumer, out):
        """``norm`` as a rider on ``producer``'s last product, if both parts around it can couple."""
        if getattr(producer, "couples_norm", False) and getattr(consumer, "couples_norm", False) and hasattr(norm, "coupling"):
            return norm.coupling(out)
        return None

    def forward(self, hidden: torch.Tensor, ctx, cache, x_in=None, next_block=None):
        """``x_in``: this block's first norm of ``hidden``, already there or carried by the block before (what that
        block returned).  ``next_block``: the block that runs next; if its first norm can ride on this block's last
        product, its input is returned, else None."""
        ws = ctx.workspace
        normed = ws.get("normed", tuple(hidden.shape), self.rt.dtype)
        if x_in is None:
            ops.stage_name = "norm"
        x = x_in if x_in is not None else self.norm1.forward(hidden, normed)
        if self.feedforward is None:
            rider = None
            if next_block is not None and getattr(next_block, "chains_norm", False):
                rider = self._rider(next_block.norm1, self.mixer, next_block.mixer, normed)
            if rider is not None:
                return self.mixer.forward(x, ctx, cache, hidden, then_norm=rider)
            self.mixer.forward(x, ctx, cache, hidden)
            return None
        rider = self._rider(self.norm2, self.mixer, self.feedforward, normed)
        x = self.mixer.forward(x, ctx, cache, hidden, then_norm=rider) if rider is not None else self.mixer.forward(x, ctx, cache, hidden)
        if x is None:
            ops.stage_name = "norm"
            x = self.norm2.forward(hidden, normed)
        rider = None
        if next_block is not None and getattr(next_block, "chains_norm", False):
            rider = self._rider(next_block.norm1, self.feedforward, next_block.mixer, normed)
        if rider is not None:
            return self.feedforward.forward(x, ctx, hidden, then_norm=rider)
        self.feedforward.forward(x, ctx, hidden)
        return None


@register_block("hyper_prenorm")
class HyperConnectionBlock(Part):
    """A pre-norm layer over ``streams`` copies ``x_1 .. x_S`` of the residual stream (hyper-connections: Zhu et al.,
    "Hyper-Connections").  Sublayer ``q`` (1: the mixer, 2: the feed-forward, where the layer has one) has learned numbers
    ``in[S]``, ``out[S]`` and ``mix[S, S]`` (indexed ``[from, to]``):

        u = sum_s in[s] x_s;   y = sublayer(norm_q(u));   x_t <- sum_s mix[s, t] x_s + out[t] y   (all streams at once).

    ``hidden`` is float32 ``[S, T, h]``.  The sublayers *add* into a float32 buffer ``y`` that the step before left zeroed,
    exactly as they add into the one residual stream of a plain block.  One kernel does a sublayer's write and the next
    sublayer's read and norm, across the border to the next block too when that is a block of this kind (``chains_norm``).
    ``block_params``: ``streams``; ``names``: ``hc1`` / ``hc2`` (the tensors' prefixes), ``in`` / ``out`` / ``mix``."""

    def __init__(self, spec: LayerSpec):
        names = spec.names
        self.streams = int(spec.block_params.get("streams", 1))
        if not 1 <= self.streams <= 8:
            raise ValueError(f"hyper_prenorm: {self.streams} streams (1 to 8)")
        norm_cls = lookup("norm", spec.norm.kind)
        self.norm1 = norm_cls(name=f"{spec.prefix}.{names['norm1']}", **spec.norm.params)
        self.mixer = lookup("mixer", spec.mixer.kind)(name=f"{spec.prefix}.{names['mixer']}", **spec.mixer.params)
        self.norm2 = self.feedforward = None
        if spec.feedforward is not None:
            self.norm2 = norm_cls(name=f"{spec.prefix}.{names['norm2']}", **spec.norm.params)
            self.feedforward = lookup("feedforward", spec.feedforward.kind)(
                name=f"{spec.prefix}.{names['feedforward']}", **spec.feedforward.params)
        for norm in (self.norm1, self.norm2):
            if norm is not None and not (hasattr(norm, "weight") and hasattr(norm, "eps") and hasattr(norm, "unit_offset")):
                raise ValueError("hyper_prenorm: the norm rides on the streams' kernel and has to be an RMS norm")
        self.hc_names = [f"{spec.prefix}.{names.get('hc1', 'hc1')}"] + ([f"{spec.prefix}.{names.get('hc2', 'hc2')}"] if self.feedforward else [])
        self.leaf = {k: names.get(k, k) for k in ("in", "out", "mix")}
        self.hc: List[Dict[str, torch.Tensor]] = []

    def parts(self) -> List[Part]:
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feedforward) if p is not None]

    def _own_specs(self) -> List[TensorSpec]:
        S = self.streams
        out = []
        for n in self.hc_names:
            out += [TensorSpec(f"{n}.{self.leaf['in']}", (S,), "bias", 1.0 / S), TensorSpec(f"{n}.{self.leaf['out']}", (S,), "bias", 1.0),
                    TensorSpec(f"{n}.{self.leaf['mix']}", (S, S), "bias", 1.0 / S)]
        return out

    def tensor_specs(self) -> List[TensorSpec]:
        return [s for p in self.parts() for s in p.tensor_specs()] + self._own_specs()

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        for p in self.parts():
            p.load(tensors, rt)
        self.hc = [{k: rt.f32(tensors.pop(f"{n}.{self.leaf[k]}")) for k in ("in", "out", "mix")} for n in self.hc_names]
        self.rt = rt

    def weight_bytes(self, dtype) -> int:
        return sum(p.weight_bytes(dtype) for p in self.parts()) + sum(spec_bytes(s, dtype) for s in self._own_specs())

    def bytes_read(self, tokens: int, dtype) -> int:
        return sum(p.bytes_read(tokens, dtype) for p in self.parts())

    def flops(self, tokens: int, pairs: int = 0) -> float:
        return sum(p.flops(tokens, pairs) for p in self.parts())

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        jobs: Dict[str, tuple] = dict(ops.library_jobs("mb_hyper"))
        for p in self.parts():
            jobs.update(p.kernel_jobs(dtype))
        return jobs

    chains_norm = True

    def _read(self, index: int, rows: torch.Tensor):
        norm = self.norm1 if index == 0 else self.norm2
        return (self.hc[index]["in"], norm.weight, norm.eps, norm.unit_offset, rows)

    def forward(self, hidden: torch.Tensor, ctx, cache, x_in=None, next_block=None):
        S, T, h = hidden.shape
        if S != self.streams:
            raise ValueError(f"hyper_prenorm: the model keeps {S} streams, the block was built for {self.streams}")
        ws = ctx.workspace
        normed = ws.get("normed", (T, h), self.rt.dtype)
        y = ws.get("sublayer_out", (T, h), torch.float32)
        if x_in is None:
            ops.stage_name = "streams, norm"
            ops.hc_step(hidden, y, read=self._read(0, normed))          # also leaves y zeroed
            x_in = normed
        self.mixer.forward(x_in, ctx, cache, y)
        last = 0
        if self.feedforward is not None:
            ops.stage_name = "streams, norm"
            ops.hc_step(hidden, y, write=(self.hc[0]["mix"], self.hc[0]["out"]), read=self._read(1, normed))
            self.feedforward.forward(normed, ctx, y)
            last = 1
        ops.stage_name = "streams, norm"
        write = (self.hc[last]["mix"], self.hc[last]["out"])
        if isinstance(next_block, HyperConnectionBlock) and next_block.streams == S:
            ops.hc_step(hidden, y, write=write, read=next_block._read(0, normed))
            return normed
        ops.hc_step(hidden, y, write=write)
        return None
