"""What a mixer asks of the cache manager.

A mixer with a growing cache asks for paged keys and values (`PagedKVNeed`); a
mixer with state of fixed size asks for a per-request slot (`SlotStateNeed`); a
mixer without memory asks for nothing.  The reference's counterpart of the first
is `DecodeStateConfig` (simply/utils/ragged_paged_attention.py:113-173); it has no
counterpart of the second (its per-request rows hold tokens and positions only,
:1451-1461).
"""

from __future__ import annotations

import dataclasses


@dataclasses.dataclass(frozen=True)
class PagedKVNeed:
  """Keys and values of every cached token, in pages.

  window: None keeps every token; an integer W keeps only what a query can still
    see, i.e. pages that lie wholly more than W-1 tokens behind the next query
    are given back.
  """

  num_kv_heads: int
  head_dim: int
  window: int | None = None


@dataclasses.dataclass(frozen=True)
class SlotStateNeed:
  """A tensor of fixed shape per live request, zeroed when the request starts."""

  shape: tuple[int, ...]
  dtype: str = "float32"
