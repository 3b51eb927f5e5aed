"""Routed feed-forward: a router picks ``top`` of ``experts`` small gated feed-forward
layers for every token.

    z = W_router h  (float32 sums; h in the activation dtype)
    s = sigmoid(z); the ``top`` experts with the largest s are chosen
    out = sum over the chosen e of expert_e(s_e * h)

The weight is the expert's score itself, not renormalised over the chosen ones, and it
multiplies the expert's INPUT (the experts are not linear, so this is not the same as
weighting their outputs).  An expert is down(act(gate x) * up x) without biases, with the
activation and its constants as parameters (the clamped form of ``ops.glu_act`` here).

Options, each a constructor parameter with the form above as its default:

``router``      "sigmoid", "softmax" over ALL router outputs, or "top_softmax": the ``top`` largest
                logits are chosen and the weights are the softmax over the chosen logits alone
``router_bias`` a vector from the checkpoint that is added to the router's logits (choice and weights)
``correction``  a vector from the checkpoint that is added to the scores for the CHOICE only
                (the weights stay the scores)
``weight_on``   "input", or "output": out = sum of s_e * expert_e(h)
``activation``  "clamped_swish" (with ``limit``) or "silu"; or "relu2": an expert WITHOUT a gate,
                down(relu(up x)^2), which has no gate matrix (``names[0]`` is not used)
``identity``    this many router outputs beyond the experts stand for experts without
                tensors whose output is their input
``shared_inner`` an expert of this inner size (same form) that every token runs, added to the sum
``groups``      (count, keep): the experts form ``count`` equal groups of neighbours; a group scores
                its best expert, and only experts of the ``keep`` best groups can be chosen
``normalize``   the weights are the chosen scores divided by their sum (+ 1e-20)
``weight_scale`` a constant on every weight
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import FeedForward, WeightSpec, register_part


class RoutedExperts(FeedForward):
    def __init__(self, width: int, inner: int, experts: int, top: int, limit: float = 0.0,
                 router_name: str = "router", expert_prefix: str = "e",
                 names=("gate", "up", "down"), router: str = "sigmoid", correction: bool = False,
                 weight_on: str = "input", activation: str = "clamped_swish", identity: int = 0,
                 shared_inner: Optional[int] = None, correction_name: str = "correction",
                 shared_prefix: str = "shared.", router_bias: bool = False,
                 router_bias_name: str = "router.b", groups=None, normalize: bool = False,
                 weight_scale: float = 1.0) -> None:
        if not 0 < top <= experts + identity:
            raise ValueError(f"top {top} of {experts} + {identity} experts")
        if router not in ops.ROUTER_KINDS or weight_on not in ("input", "output") \
                or activation not in ops.MOE_GATES + ops.MOE_PLAIN_ACTS:
            raise ValueError(f"router {router!r} / weight_on {weight_on!r} / activation {activation!r}")
        if identity and weight_on != "output":
            raise ValueError("experts without tensors need the weight on the output")
        self.groups = None
        if groups and int(groups[0]) > 1:
            count, keep = int(groups[0]), int(groups[1])
            if (experts + identity) % count or not 0 < keep <= count or top > keep * ((experts + identity) // count):
                raise ValueError(f"{count} groups of which {keep} stay do not fit top {top} of "
                                 f"{experts + identity} router outputs")
            self.groups = (count, keep)
        self.normalize, self.weight_scale = bool(normalize), float(weight_scale)
        self.width, self.inner, self.experts, self.top = width, inner, experts, top
        self.limit = float(limit)
        self.router_name, self.expert_prefix, self.names = router_name, expert_prefix, tuple(names)
        self.router, self.weight_on, self.activation = router, weight_on, activation
        self.identity, self.shared_inner = int(identity), shared_inner
        self.has_correction, self.correction_name = bool(correction), correction_name
        self.shared_prefix = shared_prefix
        self.gated = activation not in ops.MOE_PLAIN_ACTS
        self.has_router_bias, self.router_bias_name = bool(router_bias), router_bias_name
        self.router_bias = None
        self.w_router = self.w_gate_up = self.w_down = None
        self.correction = self.w_shared_gate_up = self.w_shared_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        g, u, d = self.names
        specs = {}
        for e in range(self.experts):
            p = f"{self.expert_prefix}{e}."
            if self.gated:
                specs[p + g] = WeightSpec((self.inner, self.width))
            specs[p + u] = WeightSpec((self.inner, self.width))
            specs[p + d] = WeightSpec((self.width, self.inner))
        outputs = self.experts + self.identity
        specs[self.router_name] = WeightSpec((outputs, self.width))
        if self.has_correction:
            specs[self.correction_name] = WeightSpec((outputs,), kind="vector", init="normal")
        if self.has_router_bias:
            specs[self.router_bias_name] = WeightSpec((outputs,), kind="vector", init="normal")
        if self.shared_inner:
            p = self.shared_prefix
            if self.gated:
                specs[p + g] = WeightSpec((self.shared_inner, self.width))
            specs[p + u] = WeightSpec((self.shared_inner, self.width))
            specs[p + d] = WeightSpec((self.width, self.shared_inner))
        return specs

    def kernel_libraries(self, dtype):
        return ops.linear_libraries(dtype, self.width) + ("moe",)

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u, d = self.names
        p = self.expert_prefix
        self.w_router = tensors[self.router_name].contiguous()
        first = (lambda q: torch.cat([tensors[q + g], tensors[q + u]], dim=0)) if self.gated \
            else (lambda q: tensors[q + u])
        self.w_gate_up = torch.stack([first(f"{p}{e}.") for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[f"{p}{e}.{d}"] for e in range(self.experts)]).contiguous()
        if self.has_correction:
            self.correction = tensors[self.correction_name].contiguous()
        if self.has_router_bias:
            self.router_bias = tensors[self.router_bias_name].contiguous()
        if self.shared_inner:
            p = self.shared_prefix
            self.w_shared_gate_up = first(p).contiguous()
            self.w_shared_down = tensors[p + d].contiguous()

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        logits = ops.linear_logits(x, self.w_router)          # float32 [T, router outputs]
        ids, weights = ops.moe_topk(logits, self.top, self.router, self.correction, self.router_bias,
                                    groups=self.groups, normalize=self.normalize, scale=self.weight_scale)
        base = None
        if self.shared_inner:
            if not self.gated:
                inner = ops.unary_act(ops.linear(x, self.w_shared_gate_up), self.activation)
            elif self.activation == "silu":
                inner = ops.linear_swiglu(x, self.w_shared_gate_up)
            else:
                inner = ops.glu_act(ops.linear(x, self.w_shared_gate_up), self.activation, self.limit)
            base = ops.linear(inner, self.w_shared_down)
        return ops.moe_experts(x, ids, weights, self.w_gate_up, self.w_down, self.limit,
                               gate=self.activation, weight_on=self.weight_on, identity=self.identity,
                               base=base)


register_part("feed_forward", "routed_experts", RoutedExperts)
