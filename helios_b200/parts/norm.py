"""RMSNorm (python/helios/exec/model.py:95-114): statistics in float32, no mean
subtraction, no bias.  The weight is kept in float32 in both modes."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import Norm, PendingSum, WeightSpec, register_part, settle


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, tensor_name: str = "weight") -> None:
        """``tensor_name``: the weight's name below the part's prefix ("" where the
        checkpoint names the norm itself)."""
        self.width = width
        self.eps = float(eps)
        self.tensor_name = tensor_name
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.tensor_name: WeightSpec((self.width,), kind="vector", init="ones_jitter")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.tensor_name].contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps)

    def add_forward(self, residual, delta, out_dtype, rows=None):
        if isinstance(delta, PendingSum):
            # what a block with ONE norm left pending (plain terms) rides in the norm's own launch
            if rows is None and self._plain(delta):
                (a, _), (b, _) = (delta.terms + [(None, None)] * 2)[:2]
                return ops.add_rmsnorm_pair(residual, a, b, self.weight, None, self.eps, out_dtype)[0]
            settle(residual, delta)
            delta = None
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, out_dtype, rows)

    @staticmethod
    def _plain(delta: PendingSum) -> bool:
        return delta.mult == 1.0 and len(delta.terms) <= 2 and all(s is None for _t, s in delta.terms)

    def add_forward_pair(self, residual, delta, other: "Norm", out_dtype):
        """``residual += delta`` (a tensor, a ``PendingSum`` or None), then this norm AND
        ``other`` of the new rows: (self(residual), other(residual)).  Two RMS norms with one
        eps share the row's 1 / rms, and a pending sum of plain terms rides along: one kernel."""
        if type(other) is RMSNorm and other.eps == self.eps and other.width == self.width:
            if isinstance(delta, PendingSum):
                if self._plain(delta):
                    (a, _), (b, _) = (delta.terms + [(None, None)] * 2)[:2]
                    return ops.add_rmsnorm_pair(residual, a, b, self.weight, other.weight, self.eps, out_dtype)
                settle(residual, delta)
                delta = None
            return ops.add_rmsnorm_pair(residual, delta, None, self.weight, other.weight, self.eps, out_dtype)
        first = self.add_forward(residual, delta, out_dtype)
        return first, other.add_forward(residual, None, out_dtype)

    def add_normed(self, residual, y, out_dtype):
        """``y`` None: only the residual in ``out_dtype``."""
        return ops.rmsnorm_add(residual, y, self.weight, self.eps, out_dtype)


register_part("norm", "rmsnorm", RMSNorm)


class LayerNorm(Norm):
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * weight + bias, statistics in float32; weight
    and bias stay float32 in both modes.  ``weight_name`` / ``bias_name``: the tensors' names
    below the part's prefix (the weight's may be "", where the checkpoint names the norm
    itself); ``bias=False``: no bias tensor.

    ``add_forward`` takes a ``PendingSum`` in the place of ``delta`` and does that add, scales
    and multiplier included, in the norm's own kernel."""

    def __init__(self, width: int, eps: float, weight_name: str = "weight", bias_name: str = "bias",
                 bias: bool = True) -> None:
        self.width = width
        self.eps = float(eps)
        self.weight_name, self.bias_name, self.has_bias = weight_name, bias_name, bool(bias)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {self.weight_name: WeightSpec((self.width,), kind="vector", init="ones_jitter")}
        if self.has_bias:
            specs[self.bias_name] = WeightSpec((self.width,), kind="vector", init="normal")
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()
        self.bias = tensors[self.bias_name].contiguous() if self.has_bias else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """The norm of rows in the activation dtype (statistics still float32)."""
        return ops.add_layernorm(x.float().contiguous(), self.weight, self.bias, self.eps, x.dtype)

    def add_forward(self, residual, delta, out_dtype, rows=None):
        if isinstance(delta, PendingSum):
            (a, sa), (b, sb) = (delta.terms + [(None, None)])[:2]
            return ops.add_layernorm(residual, self.weight, self.bias, self.eps, out_dtype, rows,
                                     a=a, scale_a=sa, b=b, scale_b=sb, mult=delta.mult)
        return ops.add_layernorm(residual, self.weight, self.bias, self.eps, out_dtype, rows, a=delta)


register_part("norm", "layernorm", LayerNorm)
