"""Feed-forward parts. Interface:

    FeedForward(params, weights, parts, rt)
    forward(x, out, step)     x: normed activations [T, hidden]; writes the output to out
    takes_split_norm(step)    optional, as for mixers
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import kernels
from .registry import register_part
from .runtime import Runtime, StepContext


@register_part("feed_forward", "swiglu")
class SwiGluFeedForward:
    """down(silu(gate(x)) * up(x)); gate and up are one fused projection [2I, H] (gate rows
    first), as celeg concatenates w1 and w3 (src/backend/cpu/weights_loader.cpp:93-99;
    src/backend/cuda/packed/operators.cu:531-596)."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.inner = int(params["intermediate_size"])
        self.w_gate_up = rt.matrix(torch.cat([weights["gate"], weights["up"]], dim=0))
        self.w_down = rt.matrix(weights["down"])
        self.gate_up = rt.scratch("swiglu.gate_up", 2 * self.inner)
        self.activated = rt.scratch("swiglu.act", self.inner)

    ends_with_product = True      # forward() writes `out` last, with rt.linear

    def takes_split_norm(self, step: StepContext) -> bool:
        return self.rt.takes_split_norm(step.tokens, self.w_gate_up)

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        rt, t = self.rt, step.tokens
        rt.linear_swiglu(x, self.w_gate_up, self.gate_up, self.activated, t, self.inner)
        rt.linear(self.activated, self.w_down, out, t)


@register_part("feed_forward", "dense")
class DenseFeedForward:
    """down(act(up(x))) with act one of ``gelu`` (exact, by erf), ``gelu_tanh`` or ``silu``; the activation in
    float32, rounded once."""

    ACTIVATIONS = {"gelu": kernels.ACT_GELU_ERF, "gelu_tanh": kernels.ACT_GELU_TANH, "silu": kernels.ACT_SILU}

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.inner = int(params["intermediate_size"])
        name = params.get("activation", "gelu")
        if name not in self.ACTIVATIONS:
            raise ValueError(f"dense feed-forward: unknown activation {name!r}; known: {', '.join(self.ACTIVATIONS)}")
        self.activation = self.ACTIVATIONS[name]
        self.w_up = rt.matrix(weights["up"])
        self.w_down = rt.matrix(weights["down"])
        self.raised = rt.scratch("dense.up", self.inner)

    ends_with_product = True      # forward() writes `out` last, with rt.linear

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        rt, t = self.rt, step.tokens
        rt.linear_activation(x, self.w_up, self.raised, t, self.activation)
        rt.linear(self.raised, self.w_down, out, t)
