"""Interfaces of the parts a decoder is put together from.

A part is built from its parameters alone (`PartSpec.params` plus the tensor-name
prefix); it never learns which model it is in.  It lists the tensors it needs,
takes them in `bind`, and does its work in `forward` through the kernel table
`ctx.ops`.  The roles:

* `Mixer`: mixes information between the tokens of a sequence (attention here).
  It may ask the cache manager for memory through `cache_need`.
* `FeedForward`: acts on each token alone (dense, or experts behind a router).
* `Norm`: normalises one row.
* `PositionEncoding`: gives the mixer what it needs to encode positions.
* `Block`: the arrangement of norms, mixer, feed-forward and residual adds.
* `Embedding`: token ids to the start of the residual stream.
* `Head`: the normed last hidden rows to float32 logits.

Decode steps are replayed from CUDA graphs when every part of the model says it is
`graph_safe`: its `forward` reads only the step context's device tensors (never `ctx.host`),
never waits for the device, and keeps what it prepares per step under `ctx.memo`.  What a part
prepares on the host per step (work lists) it hands to the graph runner as plans
(`Mixer.graph_plans`), which the runner keeps in a static buffer and refills between replays.

The reference's counterparts are `SimplyModule`s with `setup/init/apply`
(simply/utils/module.py:38-83); `init` is replaced by `tensor_specs` + `bind`
because weights always come from a model folder.
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.cache.needs import PagedKVNeed, SlotStateNeed
from simply_b200.config.model_spec import PartSpec
from simply_b200.weights.loader import TensorSpec


class Part:
  """Base of every part."""

  # True promises what the module's docstring asks of a part whose step is captured in a CUDA
  # graph.  The default is the safe one: a model with such a part runs its decode steps eagerly.
  graph_safe = False

  def tensor_specs(self) -> list[TensorSpec]:
    return []

  def bind(self, tensors: dict[str, torch.Tensor], ops: Any) -> None:
    """Takes this part's tensors (by full name) out of `tensors`."""


class Norm(Part):

  def apply(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    raise NotImplementedError


class PositionEncoding(Part):

  def rotation_tables(self, ctx: Any, head_dim: int) -> tuple[torch.Tensor, torch.Tensor] | None:
    """cos and sin, each f32 [T, head_dim // 2], for the step's tokens; None = no rotation."""
    raise NotImplementedError


class Mixer(Part):

  def cache_need(self) -> PagedKVNeed | SlotStateNeed | None:
    return None

  def graph_plans(self, ops: Any, batch: int, bucket: int, max_burst: int, page_size: int) -> list:
    """Plans this mixer's kernels read from `ctx.memo` in a decode step of `batch` requests with
    at most `bucket` cached tokens each, replayed up to `max_burst` times in a row.  A plan has
    `key` (its place in ctx.memo), `words` (int32 words of static device memory), `bind(view)`
    (the object to put under the key, built over that memory), `fill(host_words, lengths, steps)`
    (writes the words for a burst that starts at these lengths) and `ranges(lengths, steps)`
    (something comparable that changes whenever `fill` would write something else)."""
    return []

  def forward(self, x: torch.Tensor, ctx: Any, cache: Any, writes_cache: bool = True) -> torch.Tensor:
    """x: [T, width] in the activation dtype -> [T, width]."""
    raise NotImplementedError


class FeedForward(Part):

  def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    raise NotImplementedError


class Embedding(Part):

  vocab_size: int
  width: int

  def forward(self, ctx: Any) -> torch.Tensor:
    """float32 [T, width]: the start of the residual stream for ctx.token_ids."""
    raise NotImplementedError


class Head(Part):
  """Built with `embedding=` (the model's embedding part), which a tied output layer reads."""

  def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
    """x [R, width] (normed, activation dtype) -> float32 logits [R, vocab]."""
    raise NotImplementedError


class Block(Part):

  def cache_need(self) -> PagedKVNeed | SlotStateNeed | None:
    raise NotImplementedError

  def forward(self, stream: Any, ctx: Any, cache: Any, writes_cache: bool = True) -> None:
    """Updates the residual stream in place."""
    raise NotImplementedError


def build_part(registry, spec: PartSpec, **extra):
  """Instantiates `spec.kind` from `registry` with the spec's prefix and parameters."""
  cls = registry.get(spec.kind)
  return cls(prefix=spec.prefix, **dict(spec.params), **extra)
