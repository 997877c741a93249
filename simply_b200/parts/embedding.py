"""Token embedding and the output layer.

`token_embedding`: rows of the table times a constant, sqrt(width) for Gemma 2
(simply/utils/module.py:450-481).  `tied_head`: logits = x . table^T with the
same table, no bias, then the final soft cap (simply/model_lib.py:3183-3188,
simply/utils/module.py:416-433); logits are produced in float32.
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.parts.base import Embedding, Head
from simply_b200.registry import EMBEDDINGS, HEADS
from simply_b200.weights.loader import TensorSpec, WeightError


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):

  graph_safe = True

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


@HEADS.register("tied_head")
class TiedHead(Head):

  graph_safe = True

  def __init__(self, prefix: str, embedding: Embedding, logit_softcap: float = 0.0):
    self.embedding = embedding
    self.logit_softcap = float(logit_softcap or 0.0)

  def tensor_specs(self) -> list[TensorSpec]:
    # A folder may repeat the tied table under the output layer's name.
    return [TensorSpec("lm_head.weight", (self.embedding.vocab_size, self.embedding.width),
                       "matrix", optional=True)]

  def bind(self, tensors, ops) -> None:
    # The tied table may appear a second time under the output layer's name, but only as a copy.
    duplicate = tensors.get("lm_head.weight")
    if duplicate is not None:
      table = tensors[self.embedding.name]
      if duplicate.shape != table.shape or not torch.equal(duplicate.to(table.dtype), table):
        raise WeightError([], [], [], [], other=[
            f"lm_head.weight differs from {self.embedding.name}: this model ties its output layer to "
            "the embedding table, so the folder may repeat the table but not hold another one"])

  def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    return ctx.ops.lm_head(x, self.embedding.table, self.logit_softcap)
