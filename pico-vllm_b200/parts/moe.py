"""Routed experts: every token goes through ``top`` of ``experts`` small gated feed-forwards.

    z = W_r h + b_r  (float32)        chosen = the top largest z        weight = softmax over the chosen z alone
    y = sum over chosen e of weight_e * W_down[e] ( act(W_gate[e] h) * (W_up[e] h) ),   act = silu

Router, choice, listing of tokens per expert, both products (grouped over the experts' token lists) and the
weighted sum run on the device without a look from the host.
"""
from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..errors import ConfigError
from .base import Param, Part, Piece
from .registry import register


@register("feed_forward", "routed_experts")
class RoutedExperts(Part):
    def __init__(self, width: int, inner: int, experts: int, top: int, act: str = "silu", router_bias: bool = True):
        if act != "silu":
            raise ConfigError(f"routed_experts: activation {act!r} is not built (only 'silu')")
        if not 1 <= top <= experts or top > 32:
            raise ConfigError(f"routed_experts: top {top} must lie in 1..min(experts, 32) (experts: {experts})")
        self.width, self.inner, self.experts, self.top, self.has_bias = width, inner, experts, top, router_bias
        self.router_weight = self.router_bias = self.gate_up_weight = self.down_weight = None

    def params(self) -> List[Param]:
        gate_up, down = [], []
        for e in range(self.experts):
            gate_up += [Piece(f"e{e}.gate.weight", (self.inner, self.width)), Piece(f"e{e}.up.weight", (self.inner, self.width))]
            down.append(Piece(f"e{e}.down.weight", (self.width, self.inner)))
        ps = [Param("router_weight", (Piece("router.weight", (self.experts, self.width)),), kind="vector"),
              Param("gate_up_weight", tuple(gate_up)), Param("down_weight", tuple(down))]
        if self.has_bias:
            ps.append(Param("router_bias", (Piece("router.bias", (self.experts,)),), kind="vector"))
        return ps

    def assign(self, attr: str, tensor: torch.Tensor) -> None:
        if attr == "gate_up_weight":
            tensor = tensor.view(self.experts, 2 * self.inner, self.width)
        elif attr == "down_weight":
            tensor = tensor.view(self.experts, self.width, self.inner)
        setattr(self, attr, tensor)

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        idx, wgt = ops.moe_route(h, self.router_weight, self.router_bias, self.top)
        return ops.moe_experts(h, idx, wgt, self.gate_up_weight, self.down_weight)
