"""Token embedding and output head (python/helios/exec/model.py:419,424,486,493-496)."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import InputStage, Norm, OutputStage, Part, PositionEncoding, WeightSpec, register_part


class TokenEmbedding(InputStage):
    """hidden = table[token ids] * scale (``scale`` 1: none); no position term.  The residual
    stream it starts is float32, and so is the product."""

    def __init__(self, vocab: int, width: int, tensor_name: str = "weight", scale: float = 1.0) -> None:
        self.scale = float(scale)
        self.vocab = vocab
        self.vocab_size = vocab
        self.width = width
        self.tensor_name = tensor_name
        self.table = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.tensor_name: WeightSpec((self.vocab, self.width))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.tensor_name].contiguous()

    def forward(self, ctx) -> torch.Tensor:
        return ops.embedding(ctx.token_ids, self.table, self.scale)


class OutputHead(Part):
    """logits = rows x W^T, float32, without a bias."""

    def __init__(self, vocab: int, width: int, tensor_name: str = "weight") -> None:
        self.vocab = vocab
        self.width = width
        self.tensor_name = tensor_name
        self.weight = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.tensor_name: WeightSpec((self.vocab, self.width))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.tensor_name].contiguous()

    def kernel_libraries(self, dtype):
        return ops.linear_libraries(dtype)

    def forward(self, ctx, rows: torch.Tensor) -> torch.Tensor:
        return ops.linear_logits(rows, self.weight)


class NormedHead(OutputStage):
    """The usual end of a decoder: the last pending add and the final norm on the wanted rows
    only, then the projection to the vocabulary (python/helios/exec/model.py:491-496 norms
    every row and then selects)."""

    def __init__(self, norm: Norm, head: Part, norm_prefix: str = "model.norm.",
                 head_prefix: str = "lm_head.") -> None:
        self.norm = norm
        self.head = head
        self.norm_prefix = norm_prefix
        self.head_prefix = head_prefix

    @property
    def graph_safe(self) -> bool:
        return self.norm.graph_safe and self.head.graph_safe

    def named_parts(self):
        return [(self.norm_prefix, self.norm), (self.head_prefix, self.head)]

    def forward(self, ctx, residual: torch.Tensor, delta) -> torch.Tensor:
        rows = self.norm.add_forward(residual, delta, ctx.act_dtype, rows=ctx.want_rows)
        return self.head.forward(ctx, rows)


class LearnedPositions(PositionEncoding):
    """A learned vector per position, added (unscaled, in float32) to the embedded tokens:
    hidden[t] += table[position of t].  Positions count from 0 in every request and stay
    below ``max_positions``: the step function refuses a request that would pass it."""

    def __init__(self, max_positions: int, width: int, tensor_name: str = "weight") -> None:
        self.max_positions = max_positions
        self.width = width
        self.tensor_name = tensor_name
        self.table = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.tensor_name: WeightSpec((self.max_positions, self.width))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.tensor_name].contiguous()

    def embed(self, ctx, hidden: torch.Tensor) -> torch.Tensor:
        # the engine keeps every request below ``max_positions`` (``PositionEncoding.max_positions``)
        return ops.add_table_rows(hidden, self.table, ctx.positions)


register_part("position_encoding", "learned", LearnedPositions)
