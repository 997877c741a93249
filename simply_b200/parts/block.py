"""Block arrangements and the residual stream they act on.

The residual stream is kept in float32 whatever the activation dtype.  A branch
is not added at once: it stays *pending* together with its post-norm until the
next reader of the stream asks for a normed view.  Then one fused kernel adds
norm_post(branch) to the stream and norms the sum for the reader, so the stream
is read and written once per branch.

`sandwich_norm` is the reference's block with use_pre_ln and use_post_ln
(simply/model_lib.py:2659-2708; simply/config_lib.py:868-870):
  h += post_mixer_norm(mixer(pre_mixer_norm(h)))
  h += post_ff_norm(feed_forward(pre_ff_norm(h)))
`pre_norm` is the same without post norms (use_post_ln=False).
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.config.model_spec import PartSpec
from simply_b200.parts.base import Block, FeedForward, Mixer, Norm, build_part
from simply_b200.parts.norm import RMSNorm
from simply_b200.registry import BLOCKS, NORMS
from simply_b200.weights.loader import TensorSpec


class ResidualStream:
  """float32 [T, width] plus at most one branch that is still to be added."""

  def __init__(self, h: torch.Tensor):
    self.h = h
    self._branch: torch.Tensor | None = None
    self._post: Norm | None = None

  def add(self, branch: torch.Tensor, post_norm: Norm | None, ctx: Any) -> None:
    self.flush(ctx)
    self._branch, self._post = branch, post_norm

  def flush(self, ctx: Any) -> None:
    if self._branch is not None:
      self._combine(None, ctx, None)

  def normed(self, norm: Norm, ctx: Any, rows: torch.Tensor | None = None) -> torch.Tensor:
    """norm(h + pending) in the activation dtype.  With `rows`, only those rows are
    computed and returned (the stream is then left as it is: use this last)."""
    return self._combine(norm, ctx, rows)

  def _combine(self, pre: Norm | None, ctx: Any, rows: torch.Tensor | None):
    ops = ctx.ops
    branch, post = self._branch, self._post
    fusable = (post is None or isinstance(post, RMSNorm)) and (pre is None or isinstance(pre, RMSNorm))
    if fusable:
      out = ops.residual_norm(self.h, branch, post, pre, rows)
    else:
      # Norms the fused kernel does not know: compose from their own `apply`.
      if rows is not None:
        h = ops.gather_rows(self.h, rows)
        branch = ops.gather_rows(branch, rows) if branch is not None else None
      else:
        h = self.h
      if branch is not None:
        ops.add_to_residual(h, post.apply(branch, ctx) if post is not None else branch)
      out = pre.apply(h, ctx) if pre is not None else None
    if rows is None:
      self._branch = self._post = None
    return out


@BLOCKS.register("sandwich_norm")
class SandwichNormBlock(Block):

  uses_post_norms = True

  def __init__(self, prefix: str, width: int, norm: PartSpec, mixer: Mixer, feed_forward: FeedForward,
               names: dict[str, str] | None = None):
    self.prefix = prefix
    self.mixer = mixer
    self.feed_forward = feed_forward
    names = names or {}
    def make(role: str) -> Norm:
      return build_part(NORMS, PartSpec(norm.kind, f"{prefix}.{names.get(role, role)}",
                                        {"width": width, **norm.params}))
    self.pre_mixer = make("pre_mixer")
    self.pre_feed_forward = make("pre_feed_forward")
    self.post_mixer = make("post_mixer") if self.uses_post_norms else None
    self.post_feed_forward = make("post_feed_forward") if self.uses_post_norms else None

  def _norms(self) -> list[Norm]:
    return [n for n in (self.pre_mixer, self.post_mixer, self.pre_feed_forward,
                        self.post_feed_forward) if n is not None]

  def cache_need(self):
    return self.mixer.cache_need()

  @property
  def graph_safe(self) -> bool:
    return (self.mixer.graph_safe and self.feed_forward.graph_safe
            and all(n.graph_safe for n in self._norms()))

  def tensor_specs(self) -> list[TensorSpec]:
    specs = self.mixer.tensor_specs() + self.feed_forward.tensor_specs()
    for n in self._norms():
      specs += n.tensor_specs()
    return specs

  def bind(self, tensors, ops) -> None:
    self.mixer.bind(tensors, ops)
    self.feed_forward.bind(tensors, ops)
    for n in self._norms():
      n.bind(tensors, ops)

  def forward(self, stream: ResidualStream, ctx: Any, cache: Any, writes_cache: bool = True) -> None:
    y = stream.normed(self.pre_mixer, ctx)
    stream.add(self.mixer.forward(y, ctx, cache, writes_cache), self.post_mixer, ctx)
    y = stream.normed(self.pre_feed_forward, ctx)
    stream.add(self.feed_forward.forward(y, ctx), self.post_feed_forward, ctx)


@BLOCKS.register("pre_norm")
class PreNormBlock(SandwichNormBlock):

  uses_post_norms = False
