"""Grouped-query attention over the paged cache.

simply/model_lib.py:2091-2363 (paged branch :2136-2154): q/k/v projections
without bias (:2106-2110), position encoding on q and k then the query scale
(:2010-2019), keys and values appended to the paged cache, attention with a
soft cap on the scores before the mask (:621-634) over a causal, optionally
windowed range, and the output projection (:2362).  Query head n reads kv head
n // (num_heads / num_kv_heads) (:2306-2310).

`window = W` lets a query see W keys including itself; the reference's
`window_size` excludes the query, so W = window_size + 1
(simply/utils/ragged_paged_attention.py:922).
"""

from __future__ import annotations

from typing import Any

import torch

from simply_b200.cache.needs import PagedKVNeed
from simply_b200.config.model_spec import PartSpec
from simply_b200.parts.base import Mixer, build_part
from simply_b200.parts.linear import Linear, fuse_rows
from simply_b200.registry import MIXERS, POSITION_ENCODINGS
from simply_b200.weights.loader import TensorSpec


@MIXERS.register("paged_attention")
class PagedAttention(Mixer):

  def __init__(self, prefix: str, width: int, num_heads: int, num_kv_heads: int, head_dim: int,
               query_scale: float, logit_softcap: float = 0.0, window: int | None = None,
               position: PartSpec | None = None, project_kv: bool = True):
    if num_heads % num_kv_heads:
      raise ValueError(f"{prefix}: num_heads {num_heads} is no multiple of num_kv_heads {num_kv_heads}")
    self.prefix = prefix
    self.width = width
    self.num_heads = num_heads
    self.num_kv_heads = num_kv_heads
    self.head_dim = head_dim
    self.query_scale = float(query_scale)
    self.logit_softcap = float(logit_softcap or 0.0)
    self.window = window
    self.project_kv = project_kv
    self.position = build_part(POSITION_ENCODINGS, position or PartSpec("none"))
    self.q_proj = Linear(f"{prefix}.q_proj.weight", num_heads * head_dim, width)
    self.k_proj = Linear(f"{prefix}.k_proj.weight", num_kv_heads * head_dim, width)
    self.v_proj = Linear(f"{prefix}.v_proj.weight", num_kv_heads * head_dim, width)
    self.o_proj = Linear(f"{prefix}.o_proj.weight", width, num_heads * head_dim)
    self.qkv_weight: torch.Tensor | None = None

  def cache_need(self) -> PagedKVNeed:
    return PagedKVNeed(self.num_kv_heads, self.head_dim, self.window)

  @property
  def graph_safe(self) -> bool:
    return self.position.graph_safe

  def graph_plans(self, ops, batch: int, bucket: int, max_burst: int, page_size: int) -> list:
    plan = ops.attention_graph_plan(
        window=self.window, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
        batch=batch, bucket=bucket, max_burst=max_burst, page_size=page_size)
    return [plan] if plan is not None else []

  def tensor_specs(self) -> list[TensorSpec]:
    specs = [self.q_proj.spec()]
    if self.project_kv:
      specs += [self.k_proj.spec(), self.v_proj.spec()]
    return specs + [self.o_proj.spec()] + self.position.tensor_specs()

  def bind(self, tensors, ops) -> None:
    ops.check_attention(self.head_dim, self.num_heads, self.num_kv_heads)
    names = [self.q_proj.name] + ([self.k_proj.name, self.v_proj.name] if self.project_kv else [])
    # One matrix for q, k and v: one product per layer instead of three.
    self.qkv_weight = fuse_rows([tensors[n] for n in names])
    self.o_proj.bind(tensors)
    self.position.bind(tensors, ops)

  def forward(self, x: torch.Tensor, ctx: Any, cache: Any, writes_cache: bool = True) -> torch.Tensor:
    ops = ctx.ops
    if writes_cache and not self.project_kv:
      raise ValueError(f"{self.prefix}: a mixer without k/v projections cannot write a cache")
    tables = self.position.rotation_tables(ctx, self.head_dim)
    block_table = ctx.block_tables[cache.group]
    q = ops.project_rotate_store(
        x, self.qkv_weight, tables, self.query_scale, self.num_heads, self.num_kv_heads if self.project_kv else 0,
        self.head_dim, cache.storage if writes_cache else None, block_table, ctx)
    o = ops.paged_attention(
        q, cache.storage, block_table, ctx, num_heads=self.num_heads,
        num_kv_heads=cache.need.num_kv_heads, head_dim=self.head_dim,
        logit_softcap=self.logit_softcap, window=self.window)
    return self.o_proj(o, ctx)
