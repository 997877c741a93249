"""What a mixer asks of the cache manager.

A mixer with a growing cache asks for paged keys and values (`PagedKVNeed`); a
mixer with state of fixed size asks for a per-request slot (`SlotStateNeed`); a
mixer without memory asks for nothing.  The reference's counterpart of the first
is `DecodeStateConfig` (simply/utils/ragged_paged_attention.py:113-173); it has no
counterpart of the second (its per-request rows hold tokens and positions only,
:1451-1461).

Caches whose needs have the same `group_key()` share one pool of page ids and one block table
per request; the need itself says which of a request's pages may be given back
(`first_needed_page`) and how large its group's pool has to be (`pool_pages`).  A mixer with
another rule (a dilated window, a pool of its own) subclasses `PagedKVNeed` and overrides these;
the cache manager calls them and knows no rule of its own.
"""

from __future__ import annotations

import dataclasses

import numpy as np


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

  def group_key(self) -> tuple:
    """Needs with equal keys share page ids: the same pages are held, and given back together."""
    return ("window", self.window)

  def first_needed_page(self, lengths: np.ndarray, page_size: int) -> np.ndarray:
    """Per request, the first page that the query after `lengths` cached tokens can still see;
    pages before it may be given back.  The reference's rule,
    `max(kv_len - window_size, 0) // page_size` with its window_size = window - 1
    (simply/utils/ragged_paged_attention.py:437-443)."""
    lengths = np.asarray(lengths, dtype=np.int64)
    if self.window is None:
      return np.zeros_like(lengths)
    return np.maximum(lengths - (self.window - 1), 0) // page_size

  def first_needed_page_of(self, length: int, page_size: int) -> int:
    """`first_needed_page` for one request, in plain integers (the books' inner loops use it)."""
    if type(self).first_needed_page is PagedKVNeed.first_needed_page:
      return 0 if self.window is None else max(length - (self.window - 1), 0) // page_size
    return int(self.first_needed_page(np.array([length], dtype=np.int64), page_size)[0])

  def release_length(self, first_page: int, page_size: int) -> int | None:
    """The smallest number of cached tokens at which a request whose first held page is
    `first_page` has a page to give back (`first_needed_page` exceeds `first_page`), or None when
    this need cannot say (the books then ask `first_needed_page` every time).  A very large
    number means never."""
    if type(self).first_needed_page is not PagedKVNeed.first_needed_page:
      return None
    if self.window is None:
      return 1 << 62
    return (first_page + 1) * page_size + (self.window - 1)

  def pool_pages(self, *, page_size: int, max_slots: int, max_seq_len: int, all_pages: int,
                 step_tokens: int, burst_tokens: int) -> int:
    """Pages the group's pool needs so that it never runs out before a pool that keeps every
    token does (`all_pages`): every live request holds at most its window plus what one burst of
    decode steps adds, rounded up to pages with one page of slack at either end, and one step's
    prompt portions (`step_tokens` over all requests) come on top.  The reference sizes its local
    pool as batch * (ceil(window_size / page) + 1) and clips each portion to the room left
    (simply/serving/page_server.py:175-196, simply/utils/ragged_paged_attention.py:95-110, :418-434)."""
    if self.window is None:
      return all_pages
    per_slot = -(-(self.window - 1 + max(burst_tokens, 1)) // page_size) + 2
    per_slot = min(per_slot, -(-max_seq_len // page_size))
    return min(all_pages, max_slots * per_slot + -(-step_tokens // page_size))


@dataclasses.dataclass(frozen=True)
class SlotStateNeed:
  """A tensor of fixed shape per live request, zeroed when the request starts."""

  shape: tuple[int, ...]
  dtype: str = "float32"
