"""The generic decoder: embedding, layers in run order, final norm, output layer.

Built from a `ModelSpec` alone.  simply/model_lib.py:2935-3189 is the
reference's forward pass (embed :3000, blocks :3153-3167, final norm and head
:3183-3188); there the layer pattern is fixed by `block_attn_pattern`, here the
run order is a list that may repeat a layer or share a cache between calls.
Logits are computed only at the rows that are asked for (the reference
computes them for every token, :3186).
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.config.model_spec import ModelSpec
from simply_b200.parts.base import Block, build_part
from simply_b200.parts.block import ResidualStream
from simply_b200.registry import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS
from simply_b200.weights.loader import TensorSpec

# Importing the part modules registers the built-in parts.
from simply_b200.parts import attention as _attention  # noqa: F401
from simply_b200.parts import embedding as _embedding  # noqa: F401
from simply_b200.parts import feedforward as _feedforward  # noqa: F401
from simply_b200.parts import norm as _norm  # noqa: F401
from simply_b200.parts import position as _position  # noqa: F401


class DecoderModel:

  def __init__(self, spec: ModelSpec):
    spec.validate()
    self.spec = spec
    self.embedding = build_part(EMBEDDINGS, spec.embedding)
    self.blocks: dict[str, Block] = {}
    for layer in spec.layers:
      mixer = build_part(MIXERS, layer.mixer)
      feed_forward = build_part(FEED_FORWARDS, layer.feed_forward)
      self.blocks[layer.name] = build_part(BLOCKS, layer.block, mixer=mixer,
                                           feed_forward=feed_forward)
    self.final_norm = build_part(NORMS, spec.final_norm)
    self.head = build_part(HEADS, spec.head, embedding=self.embedding)
    self.cache_names = spec.cache_names()

  # ---- weights --------------------------------------------------------------
  def tensor_specs(self) -> list[TensorSpec]:
    specs = self.embedding.tensor_specs()
    for block in self.blocks.values():
      specs += block.tensor_specs()
    specs += self.final_norm.tensor_specs() + self.head.tensor_specs()
    names = [s.name for s in specs]
    if len(set(names)) != len(names):
      dup = sorted({n for n in names if names.count(n) > 1})
      raise ValueError(f"two parts claim the same tensor name(s): {dup}")
    return specs

  def bind(self, tensors: dict[str, torch.Tensor], ops: Any) -> None:
    self.embedding.bind(tensors, ops)
    for block in self.blocks.values():
      block.bind(tensors, ops)
    self.final_norm.bind(tensors, ops)
    self.head.bind(tensors, ops)

  def graph_safe(self) -> bool:
    """True if every part allows a decode step to be captured in a CUDA graph."""
    return (self.embedding.graph_safe and self.head.graph_safe and self.final_norm.graph_safe
            and all(b.graph_safe for b in self.blocks.values()))

  # ---- caches ---------------------------------------------------------------
  def cache_needs(self) -> dict[str, Any]:
    """Cache name -> need, taken from the call that writes the cache."""
    needs: dict[str, Any] = {}
    for call, cache in zip(self.spec.run_order, self.cache_names):
      need = self.blocks[call.layer].cache_need()
      if call.writes_cache:
        if cache in needs and needs[cache] != need:
          raise ValueError(f"cache {cache!r} is written by calls with different needs")
        needs[cache] = need
    for call, cache in zip(self.spec.run_order, self.cache_names):
      if not call.writes_cache:
        need, have = self.blocks[call.layer].cache_need(), needs[cache]
        same = (type(need) is type(have)) and all(
            getattr(need, f) == getattr(have, f) for f in ("num_kv_heads", "head_dim")
            if hasattr(have, f))
        if not same:
          raise ValueError(f"layer {call.layer!r} cannot read cache {cache!r}: {need} vs {have}")
        kept, wanted = getattr(have, "window", None), getattr(need, "window", None)
        if kept is not None and (wanted is None or wanted > kept):
          raise ValueError(
              f"layer {call.layer!r} wants to see {wanted or 'all'} keys of cache {cache!r}, "
              f"which keeps only a window of {kept}")
    return needs

  # ---- forward --------------------------------------------------------------
  def forward(self, ctx: Any, caches: dict[str, Any]) -> torch.Tensor | None:
    """Runs the step's tokens; returns float32 logits [R, vocab] at ctx.logit_rows."""
    stream = ResidualStream(self.embedding.forward(ctx))
    for call, cache in zip(self.spec.run_order, self.cache_names):
      self.blocks[call.layer].forward(stream, ctx, caches.get(cache), call.writes_cache)
    if ctx.logit_rows.numel() == 0:
      return None
    x = stream.normed(self.final_norm, ctx, rows=ctx.logit_rows)
    return self.head.forward(x, ctx)


def tensor_specs(spec: ModelSpec) -> list[TensorSpec]:
  return DecoderModel(spec).tensor_specs()
