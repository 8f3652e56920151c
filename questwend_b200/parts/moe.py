"""Routed experts: every token goes through the ``top`` of ``experts`` small gated feed-forwards that its router scores
highest, and their outputs are summed with the router's scores as weights."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.limits import moe_refusal
from ..weights.manifest import MATRIX, TensorSpec
from .base import FeedForward, take_weight
from .linear import kernel_modules as linear_modules, linear
from .registry import register_feed_forward


class RoutedExperts(FeedForward):
    """params: hidden_size, expert_size, experts, top, renormalize (default False: the weights are the chosen experts'
    softmax scores over ALL experts as they are), names (router; expert: a pattern with {e}; gate, up, down).

    Router logits W_router h in 32-bit sums; scores = softmax over all experts; the ``top`` largest are chosen.
    Expert e: W_down (silu(W_gate h) * (W_up h)), no biases."""

    NAMES = {"router": "router", "expert": "e{e}.", "gate": "gate", "up": "up", "down": "down"}

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.inter = int(p["hidden_size"]), int(p["expert_size"])
        self.experts, self.top = int(p["experts"]), int(p["top"])
        self.renormalize = bool(p.get("renormalize", False))
        self.names = {**self.NAMES, **dict(p.get("names", {}))}
        refusal = moe_refusal(self.experts, self.top)
        if refusal:
            raise ValueError(f"routed experts '{self.prefix}': {refusal}")

    def _expert(self, e, which):
        return self.prefix + self.names["expert"].format(e=e) + self.names[which]

    def tensors(self):
        out = [TensorSpec(self.prefix + self.names["router"], (self.experts, self.hidden), MATRIX)]
        for e in range(self.experts):
            out += [TensorSpec(self._expert(e, "gate"), (self.inter, self.hidden), MATRIX),
                    TensorSpec(self._expert(e, "up"), (self.inter, self.hidden), MATRIX),
                    TensorSpec(self._expert(e, "down"), (self.hidden, self.inter), MATRIX)]
        return out

    def bind(self, weights):
        self.w_router = weights[self.prefix + self.names["router"]]
        # the experts stacked: [E, 2F, D] (an expert's gate rows, then its up rows) and [E, D, F]
        first = weights[self._expert(0, "gate")]
        self.w_gate_up = torch.empty((self.experts, 2 * self.inter, self.hidden), dtype=first.dtype, device=first.device)
        self.w_down = torch.empty((self.experts, self.hidden, self.inter), dtype=first.dtype, device=first.device)
        for e in range(self.experts):
            self.w_gate_up[e, :self.inter].copy_(take_weight(weights, self._expert(e, "gate")))
            self.w_gate_up[e, self.inter:].copy_(take_weight(weights, self._expert(e, "up")))
            self.w_down[e].copy_(take_weight(weights, self._expert(e, "down")))

    def kernel_modules(self):
        return ("moe", *linear_modules(self.runtime.dtype))

    def forward(self, x, ctx):
        chosen, weight = ops.moe_route(linear(x, self.w_router), self.top, self.renormalize)
        if ops.moe_grouped_fits(x, self.w_gate_up):
            return ops.moe_experts_grouped(x, self.w_gate_up, self.w_down, chosen, weight)
        return ops.moe_experts(x, self.w_gate_up, self.w_down, chosen, weight)


register_feed_forward("routed_experts", RoutedExperts)
