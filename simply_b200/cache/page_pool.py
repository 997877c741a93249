"""A pool of page ids with a first-in first-out free list.

Same hand-out order as the reference's rotating `available_page_indices`
(simply/utils/ragged_paged_attention.py:164-165, allocate takes from the head
:509-511, release appends at the tail :530-535), kept on the host.
"""

from __future__ import annotations

import collections


class OutOfPages(RuntimeError):
  """A step needs more pages than the pool has free."""


class PagePool:

  def __init__(self, num_pages: int):
    if num_pages <= 0:
      raise ValueError(f"a page pool needs at least one page, got {num_pages}")
    self.num_pages = num_pages
    self._free: collections.deque[int] = collections.deque(range(num_pages))
    self._is_free = [True] * num_pages

  @property
  def num_free(self) -> int:
    return len(self._free)

  def take(self, n: int) -> list[int]:
    if n > len(self._free):
      raise OutOfPages(f"asked for {n} pages, {len(self._free)} of {self.num_pages} are free")
    pages = [self._free.popleft() for _ in range(n)]
    for p in pages:
      self._is_free[p] = False
    return pages

  def give_back(self, pages) -> None:
    for p in pages:
      if not 0 <= p < self.num_pages:
        raise ValueError(f"page id {p} is outside the pool of {self.num_pages}")
      if self._is_free[p]:
        raise ValueError(f"page {p} is given back twice")
      self._is_free[p] = True
      self._free.append(p)

  def free_pages(self) -> list[int]:
    return list(self._free)
