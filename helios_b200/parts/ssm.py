"""A recurrent mixer: a selective state-space layer with one scalar decay per head and token
(the recurrent form of the state-space duality).

One projection of the mixer's input gives [z | x | B | C | dt]: z and x are ``heads`` x
``head_dim`` wide, B and C ``groups`` x ``n_state`` (head h reads group h // (heads / groups)),
dt one value a head.  x, B and C together pass a short causal convolution over time per
channel (with a bias) and silu.  Per token and head, with dt = softplus(dt + dt_bias) and
a = exp(-exp(A_log) dt):

    S <- a S + dt B x^T          (S is [n_state, head_dim])
    y  = S^T C + D x

y (heads side by side) is multiplied by silu(z), RMS-normed in ``norm_parts`` equal parts of
the row (each by its own root mean square), multiplied by a weight per channel, and projected
out.  A request's slot holds S (float32) and the last taps - 1 inputs of the convolution;
nothing is kept per token.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import Mixer, StateSpec, WeightSpec, register_part


class SelectiveStateMixer(Mixer):
    def __init__(self, width: int, heads: int, head_dim: int, n_state: int, groups: int, taps: int,
                 norm_parts: int, eps: float,
                 names=("in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o")) -> None:
        """``eps``: of the output norm.  ``names``: the tensors' names below the part's prefix
        (input projection, convolution weight [channels, taps] and bias, dt bias, log of the
        decay rate, skip factor, norm weight, output projection)."""
        if heads % groups:
            raise ValueError(f"{heads} heads are not a multiple of {groups} groups")
        if taps < 1:
            raise ValueError("the convolution needs at least one tap")
        if (heads * head_dim) % norm_parts:
            raise ValueError(f"{norm_parts} norm parts do not divide {heads * head_dim} channels")
        if n_state > 256:
            raise ValueError(f"a state of {n_state} rows is not supported (at most 256)")
        self.width, self.heads, self.head_dim = width, heads, head_dim
        self.n_state, self.groups, self.taps = n_state, groups, taps
        self.norm_parts, self.eps = norm_parts, float(eps)
        self.names = tuple(names)
        self.inner = heads * head_dim
        self.conv_channels = self.inner + 2 * groups * n_state
        self.proj_rows = 2 * self.inner + 2 * groups * n_state + heads
        self.state_floats = heads * n_state * head_dim
        self.w_in = self.w_o = self.conv_w = self.conv_b = None
        self.dt_bias = self.a_log = self.d_skip = self.norm_weight = None

    def state_spec(self) -> StateSpec:
        return StateSpec((self.state_floats + self.conv_channels * (self.taps - 1),), torch.float32)

    def kernel_libraries(self, dtype):
        return ops.linear_libraries(dtype, self.width) + ("delta_rule", "ssm")

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n_in, n_conv, n_conv_b, n_dt, n_a, n_d, n_norm, n_o = self.names
        return {
            n_in: WeightSpec((self.proj_rows, self.width)),
            n_conv: WeightSpec((self.conv_channels, self.taps), kind="vector", std=0.3),
            n_conv_b: WeightSpec((self.conv_channels,), kind="vector", std=0.1),
            n_dt: WeightSpec((self.heads,), kind="vector", std=0.5),
            n_a: WeightSpec((self.heads,), kind="vector", std=0.5),
            n_d: WeightSpec((self.heads,), kind="vector", init="ones_jitter"),
            n_norm: WeightSpec((self.inner,), kind="vector", init="ones_jitter"),
            n_o: WeightSpec((self.width, self.inner)),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        n_in, n_conv, n_conv_b, n_dt, n_a, n_d, n_norm, n_o = self.names
        w = tensors[n_in]
        pad = -w.shape[0] % 8       # rows of the projection's output stay 16-byte aligned
        if pad:
            w = torch.cat([w, torch.zeros((pad, self.width), dtype=w.dtype, device=w.device)], dim=0)
        self.w_in, self.w_o = w.contiguous(), tensors[n_o].contiguous()
        self.conv_w, self.conv_b = tensors[n_conv].contiguous(), tensors[n_conv_b].contiguous()
        self.dt_bias, self.a_log = tensors[n_dt].contiguous(), tensors[n_a].contiguous()
        self.d_skip, self.norm_weight = tensors[n_d].contiguous(), tensors[n_norm].contiguous()

    def forward(self, ctx, x: torch.Tensor, cache, state: torch.Tensor) -> torch.Tensor:
        inner, gn, C = self.inner, self.groups * self.n_state, self.conv_channels
        proj = ops.linear(x, self.w_in)
        xbc = ops.causal_conv_silu(ctx, proj, C, self.conv_w, state[:, self.state_floats:],
                                   bias=self.conv_b, col0=inner)
        y = ops.ssm_scan(ctx, xbc, (0, inner, inner + gn), proj[:, inner + C:inner + C + self.heads],
                         self.a_log, self.dt_bias, self.d_skip, state[:, :self.state_floats], self.heads,
                         self.groups, self.n_state, self.head_dim)
        gated = ops.gated_group_rmsnorm(y, proj[:, :inner], self.norm_weight, self.norm_parts, self.eps)
        return ops.linear(gated, self.w_o)


register_part("mixer", "selective_state", SelectiveStateMixer)
