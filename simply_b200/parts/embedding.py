"""Token embedding and the output layer.

`token_embedding`: rows of the table times a constant, sqrt(width) for Gemma 2
(simply/utils/module.py:450-481).  `tied_head`: logits = x . table^T with the
same table, no bias, then the final soft cap (simply/model_lib.py:3183-3188,
simply/utils/module.py:416-433); logits are produced in float32.
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.parts.base import Part
from simply_b200.weights.loader import TensorSpec


class TokenEmbedding(Part):

  def __init__(self, prefix: str, vocab_size: int, width: int, scale: float = 1.0):
    self.name = f"{prefix}.weight"
    self.vocab_size = vocab_size
    self.width = width
    self.scale = float(scale)
    self.table: torch.Tensor | None = None

  def tensor_specs(self) -> list[TensorSpec]:
    return [TensorSpec(self.name, (self.vocab_size, self.width), "matrix")]

  def bind(self, tensors, ops) -> None:
    self.table = tensors[self.name]

  def forward(self, ctx: Any) -> torch.Tensor:
    """float32 [T, width]: the start of the residual stream."""
    return ctx.ops.embed(self.table, ctx.token_ids, self.scale)


class TiedHead(Part):

  def __init__(self, prefix: str, embedding: TokenEmbedding, logit_softcap: float = 0.0):
    self.embedding = embedding
    self.logit_softcap = float(logit_softcap or 0.0)

  def tensor_specs(self) -> list[TensorSpec]:
    # A folder may repeat the tied table under the output layer's name.
    return [TensorSpec("lm_head.weight", (self.embedding.vocab_size, self.embedding.width),
                       "matrix", optional=True)]

  def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    return ctx.ops.lm_head(x, self.embedding.table, self.logit_softcap)
