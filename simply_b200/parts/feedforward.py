"""Gated feed-forward: down(act(gate(x)) * up(x)), no biases.

simply/model_lib.py:714-730 with use_gated_activation_in_ffn: the activation
acts on the gate projection (`ffn_0_gate`), the product with `ffn_0` (up) feeds
`ffn_1` (down).  The activation is chosen by name; `gelu_tanh` is
simply/model_lib.py:93-96.
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.parts.base import FeedForward
from simply_b200.parts.linear import Linear, fuse_rows
from simply_b200.registry import ACTIVATIONS, FEED_FORWARDS
from simply_b200.weights.loader import TensorSpec

# Activation name -> code the gated-activation kernel takes.
ACTIVATIONS.register("gelu_tanh", 0)
ACTIVATIONS.register("silu", 1)
ACTIVATIONS.register("relu", 2)


@FEED_FORWARDS.register("gated")
class GatedFeedForward(FeedForward):

  graph_safe = True

  def __init__(self, prefix: str, width: int, hidden: int, activation: str):
    self.prefix = prefix
    self.width = width
    self.hidden = hidden
    self.activation = ACTIVATIONS.get(activation)
    self.gate_proj = Linear(f"{prefix}.gate_proj.weight", hidden, width)
    self.up_proj = Linear(f"{prefix}.up_proj.weight", hidden, width)
    self.down_proj = Linear(f"{prefix}.down_proj.weight", width, hidden)
    self.gate_up_weight: torch.Tensor | None = None

  def tensor_specs(self) -> list[TensorSpec]:
    return [self.gate_proj.spec(), self.up_proj.spec(), self.down_proj.spec()]

  def bind(self, tensors, ops) -> None:
    # Gate rows first, up rows second: one product yields [T, 2 * hidden].
    self.gate_up_weight = fuse_rows([tensors[self.gate_proj.name], tensors[self.up_proj.name]])
    self.down_proj.bind(tensors)

  def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    ops = ctx.ops
    z = ops.gated_linear(x, self.gate_up_weight, self.activation)
    return self.down_proj(z, ctx)
