"""Token embedding and output head."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import Part, Runtime, element_size
from .registry import register_embedding, register_head
from .spec import TensorSpec


@register_embedding("token_table")
class TokenEmbedding(Part):
    """``hidden[t] = float32(table[ids[t]])`` — no scaling (crates/model/src/qwen3/model.rs:133-153).  With ``positions``
    (a number of rows) a learned position table is added as it is: ``+ float32(pos_table[p])`` for the token at position
    ``p`` of its sequence.  ``tensor`` / ``position_tensor`` name the tensors where they are not ``<name>.weight``.  ``scale``
    multiplies the table's rows (in float32, as they enter the residual stream); a head tied to the table reads it unscaled."""

    def __init__(self, vocab: int, hidden: int, name: str, tensor: Optional[str] = None, positions: int = 0,
                 position_tensor: Optional[str] = None, scale: float = 1.0):
        self.vocab, self.hidden, self.name = int(vocab), int(hidden), name
        self.scale = float(scale)
        self.tensor = tensor or f"{name}.weight"
        self.positions = int(positions)
        self.position_tensor = position_tensor or f"{name}.positions.weight"
        self.table: Optional[torch.Tensor] = None
        self.pos_table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [TensorSpec(self.tensor, (self.vocab, self.hidden), "table")]
        if self.positions:
            specs.append(TensorSpec(self.position_tensor, (self.positions, self.hidden), "table"))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.table = rt.matrix(tensors.pop(self.tensor))
        if self.positions:
            self.pos_table = rt.matrix(tensors.pop(self.position_tensor))

    def bytes_read(self, tokens: int, dtype: torch.dtype) -> int:
        # only the rows asked for leave memory
        return tokens * self.hidden * element_size(dtype) * (2 if self.positions else 1)

    def forward(self, ids: torch.Tensor, out: torch.Tensor, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.positions:
            if positions is None:
                raise ValueError("an embedding with a position table needs the tokens' positions")
            ops.embed(ids, self.table, out, self.pos_table, positions, scale=self.scale)
        else:
            ops.embed(ids, self.table, out, scale=self.scale)
        return out


@register_head("linear")
class LinearHead(Part):
    """``logits = rows W^T`` in float32; ``tied_to`` names the embedding whose table is the
    head matrix when the checkpoint has no ``lm_head`` (model.rs:125-127).  ``softcap`` (a positive number) bounds the
    logits: ``cap * tanh(logits / cap)``.  ``tensor`` names the matrix where it is not ``<name>.weight``."""

    def __init__(self, vocab: int, hidden: int, name: str, tied: bool = False, softcap: Optional[float] = None,
                 tensor: Optional[str] = None):
        self.vocab, self.hidden, self.name, self.tied = int(vocab), int(hidden), name, bool(tied)
        self.softcap = float(softcap) if softcap else None
        self.tensor = tensor or f"{name}.weight"
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [] if self.tied else [TensorSpec(self.tensor, (self.vocab, self.hidden), "table")]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        if not self.tied:
            self.weight = rt.matrix(tensors.pop(self.tensor))

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table

    def bytes_read(self, tokens: int, dtype: torch.dtype) -> int:
        return self.vocab * self.hidden * element_size(dtype)      # tied or not, the whole matrix is read

    def flops(self, tokens: int, pairs: int = 0) -> float:
        """``tokens`` counts the rows whose logits are wanted."""
        return 2.0 * tokens * self.vocab * self.hidden

    def forward(self, rows: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        ops.gemm(rows, self.weight, out)
        if self.softcap is not None:
            ops.tanh_cap(out, self.softcap)
        return out
