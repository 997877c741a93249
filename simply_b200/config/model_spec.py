"""Architecture-neutral description of a decoder: parts, layers and run order.

A `ModelSpec` is plain data.  It names every part by its registry key and
gives the part its sizes and constants as parameters, layer by layer, so one
model may use different mixers and feed-forwards in different layers.  The
order in which layers run is data as well (`run_order`): an entry may name a
layer twice (the weights are reused, each call gets a cache of its own) or may
point a layer at the cache another call writes.

The reference expresses the same idea with one flat experiment config plus
`block_attn_pattern` (simply/config_lib.py:239-506, simply/model_lib.py:2839-2844);
here an architecture's config class translates its own config.json into this
neutral form and the generic builder (simply_b200/parts/model.py) does the rest.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Mapping


@dataclasses.dataclass(frozen=True)
class PartSpec:
  """One part: registry key, tensor-name prefix and its parameters."""

  kind: str
  prefix: str = ""
  params: Mapping[str, Any] = dataclasses.field(default_factory=dict)


@dataclasses.dataclass(frozen=True)
class LayerSpec:
  """One layer: a block arrangement holding a mixer and a feed-forward."""

  name: str
  block: PartSpec
  mixer: PartSpec
  feed_forward: PartSpec


@dataclasses.dataclass(frozen=True)
class LayerCall:
  """One entry of the run order.

  layer: name of the LayerSpec to run.
  cache: name of the cache this call uses.  None means a cache of its own
    (named "<layer>#<index in run order>").  Naming another call's cache makes
    this call read (and, if `writes_cache`, also extend) that cache.
  writes_cache: False for a call that only reads a cache another call wrote.
  """

  layer: str
  cache: str | None = None
  writes_cache: bool = True


@dataclasses.dataclass(frozen=True)
class ModelSpec:
  architecture: str
  vocab_size: int
  width: int
  max_context: int
  embedding: PartSpec
  layers: tuple[LayerSpec, ...]
  run_order: tuple[LayerCall, ...]
  final_norm: PartSpec
  head: PartSpec

  def layer(self, name: str) -> LayerSpec:
    for l in self.layers:
      if l.name == name:
        return l
    raise KeyError(f"run order names layer {name!r}, which the model does not define")

  def cache_names(self) -> list[str]:
    """Cache name of every call, in run order."""
    return [c.cache or f"{c.layer}#{i}" for i, c in enumerate(self.run_order)]

  def validate(self) -> None:
    names = [l.name for l in self.layers]
    if len(set(names)) != len(names):
      raise ValueError("layer names must be unique")
    if not self.run_order:
      raise ValueError("run order is empty")
    written: set[str] = set()
    for call, cache in zip(self.run_order, self.cache_names()):
      self.layer(call.layer)
      if call.writes_cache:
        written.add(cache)
      elif cache not in written:
        raise ValueError(
            f"layer call {call.layer!r} only reads cache {cache!r}, "
            "but no earlier call writes it")
