"""RMS normalisation with an optional (1 + w) scale.

simply/model_lib.py:154-178 with use_bias=False: `x * rsqrt(mean(x^2) + eps) * (1 + scale)`,
the mean of squares and the rsqrt in float32.  `plus_one` is the reference's
`scale_plus_one` (simply/config_lib.py:296).
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.parts.base import Norm
from simply_b200.registry import NORMS
from simply_b200.weights.loader import TensorSpec


@NORMS.register("rms_norm")
class RMSNorm(Norm):

  graph_safe = True

  def __init__(self, prefix: str, width: int, eps: float, plus_one: bool = True):
    self.name = f"{prefix}.weight"
    self.width = width
    self.eps = float(eps)
    self.plus_one = bool(plus_one)
    self.weight: torch.Tensor | None = None

  def tensor_specs(self) -> list[TensorSpec]:
    return [TensorSpec(self.name, (self.width,), "scale")]

  def bind(self, tensors, ops) -> None:
    self.weight = tensors[self.name]

  def apply(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    return ctx.ops.rms_norm(x, self.weight, self.eps, self.plus_one)
