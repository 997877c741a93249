"""The scheduler's decisions, with the model replaced by a rule that names the next token."""

import numpy as np
import pytest

from simply_b200.cache import CacheManager, PagedKVNeed
from simply_b200.engine.scheduler import Scheduler, Status
from simply_b200.sampling import SamplingParams


def make(pages=64, page=4, slots=4, budget=16, max_len=64, window=8, eos=()):
  cache = CacheManager({"g": PagedKVNeed(1, 8, None), "l": PagedKVNeed(1, 8, window)}, page_size=page,
                       max_slots=slots, max_seq_len=max_len, max_cache_tokens=pages * page, device=None)
  return cache, Scheduler(cache, max_num_issue_tokens=budget, max_seq_len=max_len, eos_ids=eos)


def run_step(cache, sched, next_token=lambda r: 7):
  """What the engine does around one step: plan, make room, 'run', commit."""
  plan = sched.schedule()
  assert len({e.request.slot for e in plan.entries}) == len(plan.entries)
  assert sum(e.num_tokens for e in plan.entries) <= sched.max_num_issue_tokens
  if plan.entries:
    cache.extend([(e.request.slot, e.num_tokens) for e in plan.entries])  # must never lack a page
  sampled = {e.request.request_id: next_token(e.request) for e in plan.entries if e.samples}
  finished = sched.commit(plan, sampled)
  cache.check_invariants()
  return plan, finished


def shape(plan):
  return [(e.request.request_id, e.num_tokens, e.samples) for e in plan.entries]


GREEDY = SamplingParams(temperature=0.0, max_decode_steps=4)


def test_older_first_and_the_last_one_cut():
  # After simply/utils/ragged_paged_attention_test.py:758-790: the older request takes what it
  # needs, the younger is cut to what the budget leaves.
  cache, s = make(budget=8)
  s.add("old", list(range(7)), GREEDY)
  s.add("young", list(range(3)), GREEDY)
  plan, _ = run_step(cache, s)
  assert shape(plan) == [("old", 7, True), ("young", 1, False)]
  plan, _ = run_step(cache, s)
  # decoding requests go first, then the rest of the younger prompt (its last portion samples)
  assert shape(plan) == [("old", 1, True), ("young", 2, True)]
  plan, _ = run_step(cache, s)
  assert shape(plan) == [("old", 1, True), ("young", 1, True)]


def test_budget_and_slots_limit_admission():
  cache, s = make(slots=2, budget=5)
  for i in range(3):
    s.add(i, [1] * 4, GREEDY)
  plan, _ = run_step(cache, s)
  assert shape(plan) == [(0, 4, True), (1, 1, False)]
  assert [r.request_id for r in s.waiting] == [2]  # no slot left
  assert sum(e.num_tokens for e in plan.entries) <= 5


def test_finish_reasons_and_freeing():
  cache, s = make(eos=(9,), max_len=12)
  a = s.add("eos", [1, 2, 3], SamplingParams(temperature=0, max_decode_steps=10))
  b = s.add("steps", [1, 2, 3], SamplingParams(temperature=0, max_decode_steps=2))
  c = s.add("len", [1] * 10, SamplingParams(temperature=0, max_decode_steps=10))
  d = s.add("own_stop", [1, 2], SamplingParams(temperature=0, max_decode_steps=10, stop_token_ids=(7,)))
  tokens = {"eos": iter([5, 9, 5]), "steps": iter([5, 5, 5]), "len": iter([5] * 5), "own_stop": iter([9, 7])}
  for _ in range(6):
    run_step(cache, s, lambda r: next(tokens[r.request_id]))
  assert (a.finish_reason, a.output) == ("eos", [5, 9])
  assert (b.finish_reason, b.output) == ("max_decode_steps", [5, 5])
  assert (c.finish_reason, len(c.tokens)) == ("max_seq_len", 12)
  assert (d.finish_reason, d.output) == ("eos", [9, 7])  # its own stop ids replace the model's
  assert not s.has_unfinished() and cache.num_free_slots == 4
  assert cache.all_pages_free()


def test_bad_requests_end_at_once():
  cache, s = make(max_len=8)
  assert s.add("empty", [], GREEDY).finish_reason == "empty_prompt"
  assert s.add("long", [1] * 8, GREEDY).finish_reason == "prompt_too_long"
  assert not s.has_unfinished()


def test_cancel_frees_slot_and_pages():
  cache, s = make()
  s.add("a", [1] * 10, GREEDY)
  s.add("b", [1] * 10, GREEDY)
  run_step(cache, s)
  assert s.cancel("a") and not s.cancel("nobody")
  assert cache.num_free_slots == 3
  run_step(cache, s)
  cache.check_invariants()


def test_portion_is_shortened_to_the_free_pages():
  cache, s = make(pages=3, page=4, budget=64)
  s.add("a", [1] * 30, GREEDY)
  plan, _ = run_step(cache, s)
  assert shape(plan) == [("a", 12, False)]  # three pages of four, not one token more


def test_decode_takes_pages_from_the_youngest():
  cache, s = make(pages=4, page=4, budget=64, window=100)
  s.add("old", [1] * 7, SamplingParams(temperature=0, max_decode_steps=20))
  s.add("young", [1] * 7, SamplingParams(temperature=0, max_decode_steps=20))
  plan, _ = run_step(cache, s)
  assert shape(plan) == [("old", 7, True), ("young", 7, True)]  # 2 + 2 pages: the pool is full
  plan, _ = run_step(cache, s)  # both decode into their second page
  assert shape(plan) == [("old", 1, True), ("young", 1, True)]
  plan, _ = run_step(cache, s)  # token 9 needs a third page each: only the older one goes on
  assert [r.request_id for r in plan.preempted] == ["young"]
  assert shape(plan) == [("old", 1, True)]
  young = s.waiting[0]
  assert young.status is Status.WAITING and young.num_cached == 0 and young.num_preemptions == 1
  assert len(young.tokens) == 9  # keeps what it generated; it is recomputed later
  for _ in range(40):
    run_step(cache, s)
  assert not s.has_unfinished()
  assert cache.all_pages_free()


def test_a_request_that_can_never_fit_ends_with_out_of_pages():
  cache, s = make(pages=2, page=4, budget=64)
  r = s.add("big", [1] * 8, SamplingParams(temperature=0, max_decode_steps=5))
  for _ in range(4):
    run_step(cache, s)
  assert r.finish_reason == "out_of_pages" and r.output == [7]  # one token fit, the next page did not
  assert cache.all_pages_free() and cache.num_free_slots == 4


@pytest.mark.parametrize("seed", range(5))
def test_random_load_on_a_tiny_pool_finishes_and_loses_nothing(seed):
  rng = np.random.default_rng(seed)
  cache, s = make(pages=12, page=4, slots=3, budget=int(rng.integers(2, 20)), max_len=40, window=6)
  reqs = [s.add(i, [1] * int(rng.integers(1, 30)), SamplingParams(temperature=0, max_decode_steps=int(rng.integers(1, 12))))
          for i in range(12)]
  steps = 0
  while s.has_unfinished():
    plan, _ = run_step(cache, s)
    steps += 1
    assert steps < 2000, "the scheduler does not make progress"
  assert all(r.status is Status.FINISHED for r in reqs)
  assert all(r.finish_reason in ("max_decode_steps", "max_seq_len", "out_of_pages") for r in reqs)
  assert cache.all_pages_free() and cache.num_free_slots == 3


def test_a_window_pool_smaller_than_the_full_pool():
  """The window group's pool is its own (and here deliberately scarce): the scheduler cuts portions
  and preempts by the group that is short, and every request still ends with all pages back."""
  cache = CacheManager({"g": PagedKVNeed(1, 8, None), "l": PagedKVNeed(1, 8, 8)}, page_size=4, max_slots=4,
                       max_seq_len=64, max_cache_tokens=64 * 4, device=None, step_tokens=16,
                       windowed_cache_tokens=10 * 4)
  assert [g.pool.num_pages for g in cache.groups] == [64, 10]
  s = Scheduler(cache, max_num_issue_tokens=16, max_seq_len=64)
  reqs = [s.add(i, list(range(3 + 9 * i)), SamplingParams(temperature=0.0, max_decode_steps=12)) for i in range(5)]
  for _ in range(400):
    if not s.has_unfinished():
      break
    run_step(cache, s)
  assert all(r.status is Status.FINISHED and r.finish_reason == "max_decode_steps" for r in reqs)
  assert cache.all_pages_free() and cache.num_free_slots == 4
