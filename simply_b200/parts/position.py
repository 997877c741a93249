"""Position encodings.  A position encoding hands the mixer rotation tables.

`rotary` is simply/utils/position_encoding.py:53-110: the two halves of a head
rotate together, timescale_j = theta ** (2j / head_dim), angle = position /
timescale / scale_factor, all in float32.  `none` rotates nothing.
"""

from __future__ import annotations

from typing import Any

import numpy as np
import torch

from simply_b200.parts.base import PositionEncoding
from simply_b200.registry import POSITION_ENCODINGS


@POSITION_ENCODINGS.register("rotary")
class RotaryEncoding(PositionEncoding):

  graph_safe = True

  def __init__(self, prefix: str = "", theta: float = 10000.0, scale_factor: float = 1.0):
    self.theta = float(theta)
    self.scale_factor = float(scale_factor)
    self._timescales: dict[tuple[int, str], torch.Tensor] = {}

  def timescale(self, head_dim: int, device) -> torch.Tensor:
    key = (head_dim, str(device))
    t = self._timescales.get(key)
    if t is None:
      half = head_dim // 2
      fraction = (2 * np.arange(half) / head_dim).astype(np.float32)
      t = torch.from_numpy(np.power(np.float32(self.theta), fraction).astype(np.float32)).to(device)
      self._timescales[key] = t
    return t

  def rotation_tables(self, ctx: Any, head_dim: int):
    key = ("rotary", self.theta, self.scale_factor, head_dim)
    tables = ctx.memo.get(key)
    if tables is None:
      tables = ctx.ops.rotation_tables(
          ctx.positions, self.timescale(head_dim, ctx.positions.device), self.scale_factor)
      ctx.memo[key] = tables
    return tables


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):

  graph_safe = True

  def __init__(self, prefix: str = ""):
    pass

  def rotation_tables(self, ctx: Any, head_dim: int):
    return None
