"""The cache manager's books: literal cases after the reference's own tests, then random
orders of requests with the invariants checked after every operation."""

import numpy as np
import pytest

from simply_b200.cache import CacheManager, OutOfPages, PagedKVNeed, PagePool, SlotStateNeed


def manager(window=None, page=4, pages=9, slots=3, max_len=64, extra=None):
  needs = {"kv": PagedKVNeed(2, 8, window)}
  needs.update(extra or {})
  return CacheManager(needs, page_size=page, max_slots=slots, max_seq_len=max_len,
                      max_cache_tokens=pages * page, device=None)


def rows(m, g=0):
  return [m.groups[g].held_pages(s) for s in range(m.max_slots)]


def test_allocate_in_slot_order_from_the_head_of_the_free_list():
  # simply/utils/ragged_paged_attention_test.py:83-105: 6 pages of 3 tokens, new tokens [3, 0, 4].
  m = manager(page=3, pages=6)
  s = [m.acquire_slot(i) for i in range(3)]
  m.extend([(s[0], 3), (s[2], 4)])
  assert rows(m) == [[0], [], [1, 2]]
  assert m.groups[0].pool.free_pages() == [3, 4, 5]
  m.check_invariants()


def test_allocate_on_top_of_history():
  # simply/utils/ragged_paged_attention_test.py:107-125, lengths [3, 2, 0] + new [5, 0, 6] -> [8, 2, 6].
  m = manager(page=3, pages=7)
  s = [m.acquire_slot(i) for i in range(3)]
  m.extend([(s[0], 3), (s[1], 2)])
  m.extend([(s[0], 5), (s[2], 6)])
  assert [m.length(x) for x in s] == [8, 2, 6]
  assert [len(r) for r in rows(m)] == [3, 1, 2]
  assert m.groups[0].pool.num_free == 1
  m.check_invariants()


def test_window_release_counts():
  # simply/utils/ragged_paged_attention_test.py:501-526: pages of 4, window_size 5 (W = 6),
  # lengths [3, 8, 10]: only the third gives a page back (max(10 - 5, 0) // 4 = 1).
  m = manager(window=6, page=4, pages=9)
  s = [m.acquire_slot(i) for i in range(3)]
  m.extend([(s[0], 3), (s[1], 8), (s[2], 10)])
  assert [len(r) for r in rows(m)] == [1, 2, 3]
  g = m.groups[0]
  assert [g.plan(x, m.length(x), 1)[0] for x in s] == [0, 0, 1]
  first_of_third = rows(m)[2][0]
  m.extend([(s[2], 1)])
  assert len(rows(m)[2]) == 2 and g.tables[s[2], 0] == -1
  assert g.pool.free_pages()[-1] == first_of_third  # given back to the tail of the list
  m.check_invariants()


def test_block_table_is_indexed_by_absolute_page_number():
  m = manager(window=5, page=4, pages=6, max_len=64)
  s = m.acquire_slot("r")
  for _ in range(40):
    m.extend([(s, 1)])
    m.check_invariants()
    length = m.length(s)
    g = m.groups[0]
    # every position the last token sees is on a held page, found at position // page
    for pos in range(max(length - 5, 0), length):
      assert g.tables[s, pos // 4] >= 0
    assert len(g.held_pages(s)) <= 3
  assert m.groups[0].pool.num_free >= 3  # a window of 5 never holds more than 3 pages of 4


def test_groups_share_tables_by_window_and_states_are_zeroed():
  needs = {"l0": PagedKVNeed(1, 16, 8), "l1": PagedKVNeed(1, 16, None), "l2": PagedKVNeed(2, 32, 8),
           "s": SlotStateNeed((3,), "float32"), "none": None}
  m = CacheManager(needs, page_size=4, max_slots=2, max_seq_len=32, max_cache_tokens=64, device="cpu")
  assert len(m.groups) == 2
  assert m.paged["l0"].group == m.paged["l2"].group != m.paged["l1"].group
  assert m.paged["l2"].storage.shape == (16, 2, 2, 4, 32)
  assert m.states["s"].storage.shape == (2, 3)
  s = m.acquire_slot("a")
  m.states["s"].storage[s] = 5.0
  m.release_slot(s)
  assert m.acquire_slot("b") == s and float(m.states["s"].storage[s].abs().sum()) == 0.0


def test_out_of_pages_changes_nothing():
  m = manager(page=4, pages=3)
  a, b = m.acquire_slot("a"), m.acquire_slot("b")
  m.extend([(a, 5)])
  before = (rows(m), m.groups[0].pool.free_pages(), m.length(a), m.length(b))
  assert m.pages_short([(a, 1), (b, 9)]) == 2
  with pytest.raises(OutOfPages):
    m.extend([(a, 1), (b, 9)])
  assert before == (rows(m), m.groups[0].pool.free_pages(), m.length(a), m.length(b))
  m.extend([(a, 1), (b, 4)])
  m.check_invariants()


def test_misuse_is_refused():
  m = manager()
  s = m.acquire_slot("a")
  with pytest.raises(ValueError, match="twice in one step"):
    m.extend([(s, 1), (s, 1)])
  with pytest.raises(ValueError, match="at least one token"):
    m.extend([(s, 0)])
  with pytest.raises(ValueError, match="max_seq_len"):
    m.extend([(s, 65)])
  with pytest.raises(ValueError, match="not in use"):
    m.extend([(2, 1)])
  m.release_slot(s)
  with pytest.raises(ValueError, match="released twice"):
    m.release_slot(s)
  pool = PagePool(2)
  p = pool.take(1)
  pool.give_back(p)
  with pytest.raises(ValueError, match="given back twice"):
    pool.give_back(p)
  with pytest.raises(OutOfPages):
    pool.take(3)


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_the_books_straight(seed):
  rng = np.random.default_rng(seed)
  page = int(rng.choice([1, 4, 8]))
  window = int(rng.integers(1, 20))
  needs = {"g": PagedKVNeed(1, 8, None), "l": PagedKVNeed(1, 8, window), "l2": PagedKVNeed(2, 8, window + 3)}
  m = CacheManager(needs, page_size=page, max_slots=4, max_seq_len=96, max_cache_tokens=40 * page, device=None)
  live = {}
  for _ in range(400):
    op = rng.random()
    if op < 0.15 and m.num_free_slots:
      live[m.acquire_slot(object())] = True
    elif op < 0.25 and live:
      slot = int(rng.choice(list(live)))
      m.release_slot(slot)
      del live[slot]
    elif live:
      chosen = [int(s) for s in live if rng.random() < 0.7]
      entries = [(s, int(rng.integers(1, 12))) for s in chosen if m.length(s) < 80]
      if not entries:
        continue
      lengths = {s: m.length(s) for s, _ in entries}
      if m.pages_short(entries):
        with pytest.raises(OutOfPages):
          m.extend(entries)
        assert all(m.length(s) == lengths[s] for s, _ in entries)
      else:
        m.extend(entries)
        assert all(m.length(s) == lengths[s] + n for s, n in entries)
    m.check_invariants()
  for slot in list(live):
    m.release_slot(slot)
  m.check_invariants()
  assert all(g.pool.num_free == g.pool.num_pages for g in m.groups)


def test_a_window_group_gets_a_pool_of_its_own():
  """The layer shapes of the largest named configuration, 64 requests of 8192 tokens, pages of 64:
  the group that keeps everything needs 64 * 128 pages, the window group only what 64 windows,
  a burst of decoded tokens and one step's prompt tokens can hold (the reference's
  global_total_num_pages and local_total_num_pages, simply/serving/page_server.py:175-196)."""
  needs = {"global": PagedKVNeed(16, 128, None), "local": PagedKVNeed(16, 128, 4096)}
  m = CacheManager(needs, page_size=64, max_slots=64, max_seq_len=8192, max_cache_tokens=64 * 8192,
                   device=None, step_tokens=2048, burst_tokens=16)
  sizes = {g.window: g.pool.num_pages for g in m.groups}
  assert sizes[None] == 64 * 128
  assert sizes[4096] == 64 * (-(-(4095 + 16) // 64) + 2) + 2048 // 64 == 4320
  # full size when asked for, an explicit size when given, never more than the full pool
  full = CacheManager(needs, page_size=64, max_slots=64, max_seq_len=8192, max_cache_tokens=64 * 8192, device=None)
  assert [g.pool.num_pages for g in full.groups] == [8192, 8192]
  fixed = CacheManager(needs, page_size=64, max_slots=64, max_seq_len=8192, max_cache_tokens=64 * 8192,
                       device=None, step_tokens=2048, windowed_cache_tokens=640)
  assert {g.window: g.pool.num_pages for g in fixed.groups} == {None: 8192, 4096: 10}
  small = CacheManager(needs, page_size=64, max_slots=64, max_seq_len=8192, max_cache_tokens=6400,
                       device=None, step_tokens=2048)
  assert [g.pool.num_pages for g in small.groups] == [100, 100]
  # storage follows the group's own size
  tiny = CacheManager({"g": PagedKVNeed(1, 8, None), "l": PagedKVNeed(2, 8, 5)}, page_size=4, max_slots=2,
                      max_seq_len=64, max_cache_tokens=128, device="cpu", step_tokens=8)
  assert tiny.paged["g"].storage.shape == (32, 2, 1, 4, 8)
  assert tiny.paged["l"].storage.shape == (2 * (2 + 2) + 2, 2, 2, 4, 8)


@pytest.mark.parametrize("seed", range(6))
def test_the_window_pool_never_runs_out_before_the_full_pool(seed):
  """Steps as the scheduler makes them (prompt portions that together stay under the step's token
  budget, beside bursts of decoded tokens): whenever a step lacks pages, the group that keeps every
  token lacks them too, so the smaller window pool costs no step."""
  rng = np.random.default_rng(seed)
  page = int(rng.choice([2, 4, 16]))
  window = int(rng.integers(2, 40))
  budget, burst, slots, max_len = int(rng.integers(4, 50)), int(rng.integers(1, 9)), 5, 400
  needs = {"g": PagedKVNeed(1, 8, None), "l": PagedKVNeed(1, 8, window)}
  m = CacheManager(needs, page_size=page, max_slots=slots, max_seq_len=max_len, max_cache_tokens=slots * max_len,
                   device=None, step_tokens=budget, burst_tokens=burst)
  assert m.groups[1].pool.num_pages < m.groups[0].pool.num_pages
  live = []
  for _ in range(600):
    if m.num_free_slots and rng.random() < 0.2:
      live.append(m.acquire_slot(object()))
    if live and rng.random() < 0.05:
      m.release_slot(live.pop(int(rng.integers(len(live)))))
    entries, left = [], budget
    for s in live:
      room = max_len - m.length(s)
      if rng.random() < 0.5:  # decoding: a burst
        n = min(burst, room)
      else:  # a prompt portion out of the step's budget
        n = min(int(rng.integers(0, left + 1)), room)
        left -= n
      if n > 0:
        entries.append((s, n))
    if entries:
      short_by_group = []
      for g in m.groups:
        back = take = 0
        for s, n in entries:
          b, t = g.plan(s, m.length(s), n)
          back, take = back + b, take + t
        short_by_group.append(take - back - g.pool.num_free)
      assert short_by_group[1] <= max(short_by_group[0], 0)
      if m.pages_short(entries) == 0:
        m.extend(entries)
    for s in [s for s in live if m.length(s) >= max_len]:
      m.release_slot(s)
      live.remove(s)
    m.check_invariants()


def test_a_need_with_a_rule_of_its_own_forms_a_group_of_its_own():
  """Which pages may go back is the need's rule: a need defined here keeps the first page (a
  'sink') and a window; the manager groups, sizes and releases by asking it."""
  import dataclasses

  @dataclasses.dataclass(frozen=True)
  class KeepsEverySecondWindow(PagedKVNeed):
    def group_key(self):
      return ("coarse_window", self.window)

    def first_needed_page(self, lengths, page_size):
      # gives pages back only in runs of two
      return super().first_needed_page(lengths, page_size) // 2 * 2

  needs = {"a": PagedKVNeed(1, 8, 6), "b": KeepsEverySecondWindow(1, 8, 6)}
  m = CacheManager(needs, page_size=2, max_slots=1, max_seq_len=64, max_cache_tokens=64, device=None)
  assert len(m.groups) == 2
  s = m.acquire_slot("r")
  for _ in range(20):
    m.extend([(s, 1)])
    m.check_invariants()
  assert m.groups[0].first_page[s] == (19 - 5) // 2 and m.groups[1].first_page[s] == (19 - 5) // 2 // 2 * 2


def test_a_waiting_request_keeps_no_more_than_its_window():
  """A request that got a long portion and then waits holds window + portion tokens; the pages
  below its window go back as soon as another step has to take pages."""
  m = manager(window=6, page=4, pages=12, slots=2, max_len=64)
  a, b = m.acquire_slot("a"), m.acquire_slot("b")
  m.extend([(a, 30)])
  assert len(rows(m)[a]) == 8 and m.groups[0].pool.num_free == 4
  assert m.pages_short([(b, 24)]) == 0  # 6 pages wanted, 4 free, 6 more come back from a
  m.extend([(b, 24)])
  assert m.groups[0].first_page[a] == (30 - 5) // 4 and len(rows(m)[a]) == 2
  assert len(rows(m)[b]) == 6
  m.check_invariants()
