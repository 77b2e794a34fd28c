"""Normalisation parts."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import Part, Runtime
from .registry import register_norm
from .spec import TensorSpec


@register_norm("rmsnorm")
class RMSNorm(Part):
    """``y_i = x_i / sqrt(mean(x^2) + eps) * w_i`` over the last axis, sums in float32.

    The weight multiplies directly (no ``1 + w``), as the reference computes it
    (crates/tensor/src/norm.rs:16-22, crates/cuda/src/kernels.cu:51-58); ``unit_offset``
    selects the ``1 + w`` form other architectures use (their weights lie around zero).  ``tensor`` names the weight
    inside ``name`` where it is not ``weight`` ("" for the tensor ``name`` itself).
    """

    def __init__(self, dim: int, eps: float, name: str, unit_offset: bool = False, tensor: str = "weight"):
        self.dim, self.eps, self.name, self.unit_offset = int(dim), float(eps), name, bool(unit_offset)
        self.weight_name = f"{name}.{tensor}" if tensor else name
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.weight_name, (self.dim,), "norm", 0.0 if self.unit_offset else None)]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.weight = rt.f32(tensors.pop(self.weight_name))

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``x`` float32 ``[rows, dim]`` → ``out`` (float32 or bfloat16) ``[rows, dim]``."""
        ops.rmsnorm(x, self.weight, self.eps, out, self.unit_offset)
        return out

    def coupling(self, out: torch.Tensor) -> "ops.NormOut":
        """This norm as a rider on the product that last updates its input (``ops.gemm(..., then_norm=...)``)."""
        return ops.NormOut(self.weight, self.unit_offset, self.eps, out)


@register_norm("dynamic_tanh")
class DynamicTanh(Part):
    """``y_i = tanh(alpha * x_i) * w_i + b_i``: a norm that takes no statistic of the row (no mean, no variance), with one
    learned scalar ``alpha``.  ``eps`` is accepted like every norm's and not used.  ``names`` gives the tensors' names
    inside ``name`` (weight, bias, alpha); ``bias=False`` leaves the offset out."""

    def __init__(self, dim: int, name: str, eps: float = 0.0, bias: bool = True, names=("weight", "bias", "alpha")):
        self.dim, self.name, self.eps, self.has_bias = int(dim), name, float(eps), bool(bias)
        join = lambda part: f"{name}.{part}" if part else name     # "" names the tensor `name` itself
        self.weight_name, self.bias_name, self.alpha_name = (join(p) for p in names)
        self.weight = self.bias = self.alpha = None

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [TensorSpec(self.weight_name, (self.dim,), "norm")]
        if self.has_bias:
            specs.append(TensorSpec(self.bias_name, (self.dim,), "bias"))
        return specs + [TensorSpec(self.alpha_name, (), "norm")]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.weight = rt.f32(tensors.pop(self.weight_name))
        self.bias = rt.f32(tensors.pop(self.bias_name)) if self.has_bias else None
        self.alpha = rt.f32(tensors.pop(self.alpha_name)).reshape(1)

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``x`` float32 ``[rows, dim]`` → ``out`` (float32 or bfloat16) ``[rows, dim]``."""
        ops.dynamic_tanh(x, self.weight, self.bias, self.alpha, out)
        return out
