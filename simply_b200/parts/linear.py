"""A bias-free linear map y = x W^T with W stored [out, in].

The reference's `EinsumLinear` (simply/utils/module.py:191-355, apply :339-355)
with the projections' einsum strings flattened: its `[D, H, dh]` projection
weights (simply/model_lib.py:2037-2072) are the `[H*dh, D]` matrices of the
model folder transposed, row n*dh + d <-> w[:, n, d].
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.weights.loader import TensorSpec


class Linear:

  def __init__(self, name: str, out_features: int, in_features: int):
    self.name = name
    self.out_features = out_features
    self.in_features = in_features
    self.weight: torch.Tensor | None = None

  def spec(self) -> TensorSpec:
    return TensorSpec(self.name, (self.out_features, self.in_features), "matrix")

  def bind(self, tensors: dict[str, torch.Tensor]) -> None:
    self.weight = tensors[self.name]

  def __call__(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    return ctx.ops.linear(x, self.weight)


def fuse_rows(weights: list[torch.Tensor]) -> torch.Tensor:
  """Stacks [out_i, in] matrices into one; 32-bit wins if the dtypes differ."""
  dtype = torch.float32 if any(w.dtype == torch.float32 for w in weights) else weights[0].dtype
  return torch.cat([w.to(dtype) for w in weights], dim=0).contiguous()
