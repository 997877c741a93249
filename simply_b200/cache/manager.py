"""The cache manager: slots, page groups, block tables and per-request state.

Requests live in *slots*.  Caches with a growing need (keys and values) are
kept in pages.  Caches whose need for pages is the same (all tokens, or a
window of W tokens) form a *group*: a group has one pool of page ids, sized
for what its caches can hold at once, and one block table per slot, and a
page id is valid in the storage of every cache of its group.  Caches of fixed size per request (`SlotStateNeed`) are rows of a
tensor indexed by slot.

Bookkeeping follows the reference's `DecodeState`
(simply/utils/ragged_paged_attention.py:176-541), moved to the host:

* `extend` = `release_for_window().allocate(q_lens)` (:437-518): before a step,
  a windowed group gives back the pages that lie wholly below what the step's
  first query can see, then every group takes the pages the new tokens need.
  The count of pages to give back is `max(len - (W-1), 0) // page_size`, the
  reference's `max(kv_len - window_size, 0) // page_size` with its
  `window_size = W - 1` (:437-443).
* groups: the reference shares bookkeeping between layers with equal
  `(total_pages, page_size, window)` (:865-867, :901-917).
* `release_slot` = `release` (:521-541).

Unlike the reference the block table is indexed by the absolute page number of
a position (`position // page_size`); pages that were given back read -1.  The
kernels never follow a -1.  A step that cannot get its pages raises
`OutOfPages` before anything is changed (the reference leaves that case
undefined, :493-494).
"""

from __future__ import annotations

import dataclasses
from typing import Mapping, Sequence

import numpy as np
import torch

from simply_b200.cache.needs import PagedKVNeed, SlotStateNeed
from simply_b200.cache.page_pool import OutOfPages, PagePool


def _cdiv(a: int, b: int) -> int:
  return -(-a // b)


class PageGroup:
  """Pages and block tables of the caches that share page ids (equal `need.group_key()`).

  The group's pool has a size of its own, and which pages a request may give back is the
  need's rule (`need.first_needed_page`), not the group's."""

  def __init__(self, need: PagedKVNeed, page_size: int, num_pages: int, max_slots: int,
               max_seq_len: int):
    self.need = need
    self.window = getattr(need, "window", None)
    self.page_size = page_size
    self.num_pages = num_pages
    self.pool = PagePool(num_pages)
    self.max_pages_per_seq = _cdiv(max_seq_len, page_size)
    self.tables = np.full((max_slots, self.max_pages_per_seq), -1, dtype=np.int32)
    # Pages [first_page, end_page) of a slot are held.
    self.first_page = np.zeros(max_slots, dtype=np.int64)
    self.end_page = np.zeros(max_slots, dtype=np.int64)
    self.cache_names: list[str] = []
    self.version = 0  # counts changes of `tables`: who holds a copy can tell whether it is current

  def plan(self, slot: int, cur_len: int, n_new: int) -> tuple[int, int]:
    """(pages to give back, pages to take) for `n_new` tokens after `cur_len` cached ones."""
    first, end = int(self.first_page[slot]), int(self.end_page[slot])
    new_first = max(first, self.need.first_needed_page_of(cur_len, self.page_size))
    new_first = min(new_first, end)
    new_end = max(end, _cdiv(cur_len + n_new, self.page_size))
    return new_first - first, new_end - end

  def apply(self, slot: int, cur_len: int, n_new: int) -> tuple[list[int], list[int]]:
    """Carries out `plan`; returns (pages given back, pages taken)."""
    n_back, n_take = self.plan(slot, cur_len, n_new)
    if n_back == 0 and n_take == 0:
      return [], []  # the usual decode step: the token lands in a page the slot already holds
    self.version += 1
    first, end = int(self.first_page[slot]), int(self.end_page[slot])
    row = self.tables[slot]
    back = [int(p) for p in row[first:first + n_back]]
    self.pool.give_back(back)
    row[first:first + n_back] = -1
    self.first_page[slot] = first + n_back
    taken = self.pool.take(n_take)
    row[end:end + n_take] = taken
    self.end_page[slot] = end + n_take
    return back, taken

  def release_slot(self, slot: int) -> list[int]:
    first, end = int(self.first_page[slot]), int(self.end_page[slot])
    back = [int(p) for p in self.tables[slot, first:end]]
    self.pool.give_back(back)
    self.version += 1
    self.tables[slot, :] = -1
    self.first_page[slot] = 0
    self.end_page[slot] = 0
    return back

  def held_pages(self, slot: int) -> list[int]:
    return [int(p) for p in self.tables[slot, int(self.first_page[slot]):int(self.end_page[slot])]]


@dataclasses.dataclass
class PagedCache:
  """Handle a mixer gets for its paged cache."""

  name: str
  group: int  # index into CacheManager.groups
  need: PagedKVNeed
  # [num_pages, 2 (keys, values), num_kv_heads, page_size, head_dim]
  storage: torch.Tensor | None


@dataclasses.dataclass
class SlotState:
  """Handle a mixer gets for its per-request state: tensor [max_slots, *shape]."""

  name: str
  need: SlotStateNeed
  storage: torch.Tensor | None


class CacheManager:

  def __init__(
      self,
      needs: Mapping[str, PagedKVNeed | SlotStateNeed | None],
      *,
      page_size: int,
      max_slots: int,
      max_seq_len: int,
      max_cache_tokens: int,
      dtype: torch.dtype = torch.float32,
      device: torch.device | str | None = "cpu",
      poison_freed_pages: bool = False,
      step_tokens: int | None = None,
      burst_tokens: int = 1,
      windowed_cache_tokens: int = 0,
  ):
    """`device=None` keeps the books only (no storage), for host-side tests.

    `max_cache_tokens` sizes the pool of a group that keeps every token.  A group that gives
    pages back asks its need how many pages it can ever hold at once (`need.pool_pages`, from
    `step_tokens` prompt tokens per step over all requests and `burst_tokens` decoded tokens per
    request between two looks at the tables) and gets that many, never more than the former;
    `step_tokens=None` gives every group the full size, `windowed_cache_tokens > 0` fixes the
    size of those groups (the reference's `global_total_num_pages` and `local_total_num_pages`,
    simply/serving/page_server.py:175-196)."""
    self.page_size = page_size
    self.max_slots = max_slots
    self.max_seq_len = max_seq_len
    self.num_pages = _cdiv(max_cache_tokens, page_size)
    self.poison_freed_pages = poison_freed_pages
    self.groups: list[PageGroup] = []
    self.paged: dict[str, PagedCache] = {}
    self.states: dict[str, SlotState] = {}
    group_of_key: dict[tuple, int] = {}
    for name, need in needs.items():
      if need is None:
        continue
      if isinstance(need, PagedKVNeed):
        window = getattr(need, "window", None)
        if window is not None and window <= 0:
          raise ValueError(f"cache {name!r}: window must be positive, got {window}")
        g = group_of_key.get(need.group_key())
        if g is None:
          g = len(self.groups)
          group_of_key[need.group_key()] = g
          pages = self.num_pages
          if step_tokens is not None:
            pages = need.pool_pages(page_size=page_size, max_slots=max_slots, max_seq_len=max_seq_len,
                                    all_pages=self.num_pages, step_tokens=step_tokens,
                                    burst_tokens=burst_tokens)
            if windowed_cache_tokens > 0 and window is not None:
              pages = min(self.num_pages, _cdiv(windowed_cache_tokens, page_size))
          self.groups.append(PageGroup(need, page_size, max(pages, 1), max_slots, max_seq_len))
        self.groups[g].cache_names.append(name)
        storage = None
        if device is not None:
          storage = torch.zeros(
              (self.groups[g].num_pages, 2, need.num_kv_heads, page_size, need.head_dim),
              dtype=dtype, device=device)
        self.paged[name] = PagedCache(name, g, need, storage)
      elif isinstance(need, SlotStateNeed):
        storage = None
        if device is not None:
          storage = torch.zeros((max_slots, *need.shape), dtype=getattr(torch, need.dtype),
                                device=device)
        self.states[name] = SlotState(name, need, storage)
      else:
        raise TypeError(f"cache {name!r}: unknown kind of need {need!r}")
    self.lengths = np.zeros(max_slots, dtype=np.int64)
    # Per slot, what the usual decode step asks in one look: up to which length a step may bring
    # tokens without taking a page (the smallest group's held pages), and from which length on
    # some group has a page to give back.  Kept current by `_refresh_limits` whenever a slot's
    # pages change.  `_fast_limits` is False when a need cannot name its release length.
    self._grow_limit = [0] * max_slots
    self._release_at = [1 << 62] * max_slots
    self._fast_limits = all(g.need.release_length(0, page_size) is not None for g in self.groups)
    self.owner: list[object | None] = [None] * max_slots
    self._live = np.zeros(max_slots, dtype=bool)  # owner is not None
    self._free_slots = list(range(max_slots - 1, -1, -1))

  def _release_at_array(self) -> np.ndarray:
    return np.asarray(self._release_at, dtype=np.int64)

  def _changes_table(self, slot: int, n: int) -> bool:
    """Whether `n` more tokens take or give back a page of this slot (any group)."""
    if not self._fast_limits:
      return True
    cur = self.lengths[slot]
    return cur + n > self._grow_limit[slot] or cur >= self._release_at[slot]

  def _refresh_limits(self, slot: int) -> None:
    if not self._fast_limits:
      return
    grow, release = 1 << 62, 1 << 62
    for g in self.groups:
      grow = min(grow, int(g.end_page[slot]) * self.page_size)
      if int(g.first_page[slot]) < int(g.end_page[slot]):
        release = min(release, g.need.release_length(int(g.first_page[slot]), self.page_size))
    self._grow_limit[slot] = grow if self.groups else 1 << 62
    self._release_at[slot] = release

  # ---- slots ----------------------------------------------------------------
  @property
  def num_free_slots(self) -> int:
    return len(self._free_slots)

  def acquire_slot(self, owner: object) -> int:
    if not self._free_slots:
      raise RuntimeError("no free slot")
    slot = self._free_slots.pop()
    self.owner[slot] = owner
    self._live[slot] = True
    self.lengths[slot] = 0
    self._refresh_limits(slot)
    for s in self.states.values():
      if s.storage is not None:
        s.storage[slot].zero_()
    return slot

  def release_slot(self, slot: int) -> None:
    """Gives back every page of the slot and frees the slot."""
    if self.owner[slot] is None:
      raise ValueError(f"slot {slot} is released twice")
    for gi, g in enumerate(self.groups):
      self._poison(gi, g.release_slot(slot))
    self.owner[slot] = None
    self._live[slot] = False
    self.lengths[slot] = 0
    self._refresh_limits(slot)
    self._free_slots.append(slot)

  def length(self, slot: int) -> int:
    return int(self.lengths[slot])

  # ---- pages ----------------------------------------------------------------
  def changes_no_table(self, entries: Sequence[tuple[int, int]]) -> bool:
    """True if the batch `[(slot, new tokens)]` neither takes nor gives back a page in any group
    (the usual decode step).  One vectorised look instead of a plan per slot and group."""
    if not entries:
      return True
    if self._fast_limits:
      lengths, grow, release = self.lengths, self._grow_limit, self._release_at
      for slot, n in entries:
        cur = lengths[slot]
        if cur + n > grow[slot] or cur >= release[slot]:
          return False
      return True
    slots = np.fromiter((s for s, _ in entries), dtype=np.int64, count=len(entries))
    new = np.fromiter((n for _, n in entries), dtype=np.int64, count=len(entries))
    cur = self.lengths[slots]
    for g in self.groups:
      if np.any(-(-(cur + new) // self.page_size) > g.end_page[slots]):
        return False
      first = np.minimum(g.need.first_needed_page(cur, self.page_size), g.end_page[slots])
      if np.any(first > g.first_page[slots]):
        return False
    return True

  def _idle_releasable(self, g: PageGroup, busy: set[int]) -> list[tuple[int, int]]:
    """(slot, pages) of live requests outside the step that hold pages no later query of theirs
    can see (what their last portion left below the window).  Such pages go back whenever a step
    has to take pages, so that a request that waits never keeps more than its window."""
    if g.window is None and type(g.need) is PagedKVNeed:
      return []  # keeps every token
    if self._fast_limits and not np.any(self._live & (self.lengths >= self._release_at_array())):
      return []  # no live request at all has a page to give back
    live = self._live.copy()
    if busy:
      live[list(busy)] = False
    idx = np.nonzero(live)[0]
    if idx.size == 0:
      return []
    first = np.minimum(g.need.first_needed_page(self.lengths[idx], self.page_size), g.end_page[idx])
    extra = first - g.first_page[idx]
    return [(int(s), int(n)) for s, n in zip(idx, extra) if n > 0]

  def pages_short(self, entries: Sequence[tuple[int, int]]) -> int:
    """How many pages the batch `[(slot, new tokens)]` lacks (0 if it fits), worst group."""
    if self.changes_no_table(entries):
      return 0
    short = 0
    busy = {slot for slot, _ in entries}
    changing = [(slot, n) for slot, n in entries if self._changes_table(slot, n)]
    if len(changing) <= 16:
      for g in self.groups:
        back = sum(n for _, n in self._idle_releasable(g, busy))
        take = 0
        for slot, n in changing:
          b, t = g.plan(slot, int(self.lengths[slot]), n)
          back += b
          take += t
        short = max(short, take - back - g.pool.num_free)
      return max(short, 0)
    slots = np.fromiter((s for s, _ in changing), dtype=np.int64, count=len(changing))
    new = np.fromiter((n for _, n in changing), dtype=np.int64, count=len(changing))
    cur = self.lengths[slots]
    for g in self.groups:
      # `PageGroup.plan` for all of them at once.
      first, end = g.first_page[slots], g.end_page[slots]
      new_first = np.minimum(np.maximum(first, g.need.first_needed_page(cur, self.page_size)), end)
      new_end = np.maximum(end, -(-(cur + new) // self.page_size))
      back = int((new_first - first).sum()) + sum(n for _, n in self._idle_releasable(g, busy))
      take = int((new_end - end).sum())
      short = max(short, take - back - g.pool.num_free)
    return max(short, 0)

  def pages_needed(self, slot: int, n_new: int) -> int:
    """Net pages (taken minus given back) that `n_new` more tokens cost, worst group."""
    worst = 0
    for g in self.groups:
      b, t = g.plan(slot, int(self.lengths[slot]), n_new)
      worst = max(worst, t - b)
    return worst

  def tables_version(self) -> int:
    """Changes whenever a block table of any group changes."""
    return sum(g.version for g in self.groups)

  def min_free_pages(self) -> int:
    return min((g.pool.num_free for g in self.groups), default=1 << 30)

  def all_pages_free(self) -> bool:
    """True when no request holds a page in any group."""
    return all(g.pool.num_free == g.pool.num_pages for g in self.groups)

  def extend(self, entries: Sequence[tuple[int, int]]) -> None:
    """Makes room for the step's new tokens; all or nothing."""
    seen = set()
    for slot, n in entries:
      if self.owner[slot] is None:
        raise ValueError(f"slot {slot} is not in use")
      if slot in seen:
        raise ValueError(f"slot {slot} appears twice in one step")
      seen.add(slot)
      if n <= 0:
        raise ValueError(f"slot {slot}: a step entry needs at least one token, got {n}")
      if self.lengths[slot] + n > self.max_seq_len:
        raise ValueError(
            f"slot {slot}: {int(self.lengths[slot])} + {n} tokens exceed max_seq_len "
            f"{self.max_seq_len}")
    if self.changes_no_table(entries):
      for slot, n in entries:
        self.lengths[slot] += n
      return
    short = self.pages_short(entries)
    if short:
      raise OutOfPages(f"the step lacks {short} page(s)")
    # Only the entries whose pages change need the books; the others just grow.
    changing = [(slot, n) for slot, n in entries if self._changes_table(slot, n)]
    touched = {slot for slot, _ in changing}
    for gi, g in enumerate(self.groups):
      # Every slot gives back before any slot takes, as the pool may need those pages: first the
      # requests outside the step, then the step's own.
      for slot, _ in self._idle_releasable(g, seen):
        back, _ = g.apply(slot, int(self.lengths[slot]), 0)
        self._poison(gi, back)
        touched.add(slot)
      for slot, n in changing:
        cur = int(self.lengths[slot])
        n_back, _ = g.plan(slot, cur, 0)
        if n_back:
          back, _ = g.apply(slot, cur, 0)
          self._poison(gi, back)
      for slot, n in changing:
        g.apply(slot, int(self.lengths[slot]), n)
    for slot, n in entries:
      self.lengths[slot] += n
    for slot in touched:
      self._refresh_limits(slot)

  def _poison(self, group: int, pages: list[int]) -> None:
    if not self.poison_freed_pages or not pages:
      return
    for name in self.groups[group].cache_names:
      st = self.paged[name].storage
      if st is not None:
        st[torch.as_tensor(pages, device=st.device, dtype=torch.long)] = float("nan")

  # ---- checks ---------------------------------------------------------------
  def check_invariants(self) -> None:
    """No page lost, none held twice, tables and lengths consistent."""
    for g in self.groups:
      held: list[int] = []
      for slot in range(self.max_slots):
        pages = g.held_pages(slot)
        if self.owner[slot] is None and pages:
          raise AssertionError(f"free slot {slot} holds pages {pages}")
        if any(p < 0 for p in pages):
          raise AssertionError(f"slot {slot} holds an invalid page id in {pages}")
        row = g.tables[slot]
        outside = np.concatenate([row[:int(g.first_page[slot])], row[int(g.end_page[slot]):]])
        if (outside != -1).any():
          raise AssertionError(f"slot {slot} has page ids outside its held range")
        if self.owner[slot] is not None:
          length = int(self.lengths[slot])
          if int(g.end_page[slot]) != _cdiv(length, self.page_size):
            raise AssertionError(
                f"slot {slot}: {int(g.end_page[slot])} pages end for {length} tokens")
          if length > 0:
            # Everything the request's next query can see must still be held.
            needed = int(g.need.first_needed_page(np.array([length]), self.page_size)[0])
            if int(g.first_page[slot]) > needed:
              raise AssertionError(f"slot {slot}: pages that are still visible were given back")
        held.extend(pages)
      free = g.pool.free_pages()
      if len(set(held)) != len(held):
        raise AssertionError("a page is held twice")
      if set(held) & set(free):
        raise AssertionError("a page is both held and free")
      if len(held) + len(free) != g.pool.num_pages or len(set(free)) != len(free):
        raise AssertionError(
            f"pages lost: {len(held)} held + {len(free)} free != {g.pool.num_pages}")
