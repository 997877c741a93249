"""The scheduler: admits requests, cuts prompts into portions, decodes, finishes, frees.

Policy, after the reference's batcher and slot table
(simply/serving/page_batcher.py:701-895, simply/utils/ragged_paged_attention.py:1821-1859):
requests that are decoding go first, in order of arrival, then prompt portions
in order of arrival until the step's token budget is used; the last one is cut
to what is left (`issue_lens`, :1831-1859).  Differences: one step may mix
decoded tokens and prompt portions; the last prompt portion asks for its own
logits, so the first generated token costs no extra step (the reference stops
the prompt at `input_len - 1`, :1556-1557); a request ends on eos, on
`max_decode_steps` or at `max_seq_len` (`has_ended`, :1936-1944).

When pages run out (the reference sizes its pools so that they cannot,
simply/serving/page_server.py:175-196, and leaves the case undefined,
ragged_paged_attention.py:493-494):
  1. a prompt portion is shortened to the pages that are free, or waits;
  2. a decoding request that cannot get its page makes the youngest live
     request give up its slot and pages; that request goes back to the head of
     the queue and is later recomputed from its tokens so far (its sampling is
     keyed by position, so it continues as if nothing had happened);
  3. a request that cannot fit even alone ends with reason "out_of_pages".
No step is ever launched that needs a page it does not hold.
"""

from __future__ import annotations

import collections
import dataclasses
import enum
from typing import Sequence

from simply_b200.cache.manager import CacheManager
from simply_b200.sampling.params import SamplingParams


class Status(enum.Enum):
  WAITING = "waiting"
  RUNNING = "running"
  FINISHED = "finished"


@dataclasses.dataclass(eq=False)  # a request is itself: lists and queues look it up by identity
class Request:
  request_id: object
  prompt: list[int]
  params: SamplingParams
  arrival: int = 0
  tokens: list[int] = dataclasses.field(default_factory=list)  # prompt + generated
  num_cached: int = 0  # tokens whose keys/values are in the cache
  slot: int | None = None
  status: Status = Status.WAITING
  finish_reason: str | None = None
  num_preemptions: int = 0
  logprobs: list[float] = dataclasses.field(default_factory=list)  # of the generated tokens, if asked for

  @property
  def output(self) -> list[int]:
    return self.tokens[len(self.prompt):]

  @property
  def num_output(self) -> int:
    return len(self.tokens) - len(self.prompt)

  @property
  def remaining(self) -> int:
    return len(self.tokens) - self.num_cached

  @property
  def is_decoding(self) -> bool:
    return self.remaining == 1 and len(self.tokens) > len(self.prompt)


@dataclasses.dataclass
class PlannedEntry:
  request: Request
  num_tokens: int
  samples: bool  # the step computes the logits after this entry's last token


@dataclasses.dataclass
class StepPlan:
  entries: list[PlannedEntry]
  preempted: list[Request]
  failed: list[Request]


class Scheduler:

  def __init__(self, cache: CacheManager, *, max_num_issue_tokens: int, max_seq_len: int,
               eos_ids: Sequence[int] = ()):
    self.cache = cache
    self.max_num_issue_tokens = max_num_issue_tokens
    self.max_seq_len = max_seq_len
    self.eos_ids = tuple(eos_ids)
    self.waiting: collections.deque[Request] = collections.deque()
    self.running: list[Request] = []
    self._arrivals = 0

  # ---- admission --------------------------------------------------------------
  def add(self, request_id, prompt: Sequence[int], params: SamplingParams) -> Request:
    r = Request(request_id, list(prompt), params, arrival=self._arrivals, tokens=list(prompt))
    self._arrivals += 1
    if not r.prompt:
      self._finish(r, "empty_prompt")
    elif len(r.prompt) >= self.max_seq_len:
      # The reference keeps the last max_seq_len tokens (simply/utils/sampling_lib.py:368-369);
      # this engine refuses instead of silently dropping the start of a prompt.
      self._finish(r, "prompt_too_long")
    else:
      self.waiting.append(r)
    return r

  def has_unfinished(self) -> bool:
    return bool(self.waiting or self.running)

  def cancel(self, request_id) -> bool:
    for r in list(self.running) + list(self.waiting):
      if r.request_id == request_id:
        self._finish(r, "cancelled")
        return True
    return False

  # ---- planning ----------------------------------------------------------------
  def schedule(self) -> StepPlan:
    plan = StepPlan([], [], [])
    budget = self.max_num_issue_tokens
    chosen: list[tuple[int, int]] = []  # (slot, tokens) of the entries so far

    def fits(slot: int, n: int) -> bool:
      return self.cache.pages_short(chosen + [(slot, n)]) == 0

    def largest_fitting(slot: int, n: int) -> int:
      if fits(slot, n):
        return n
      lo, hi = 0, n  # fits(lo) (vacuously for 0), not fits(hi)
      while hi - lo > 1:
        mid = (lo + hi) // 2
        if fits(slot, mid):
          lo = mid
        else:
          hi = mid
      return lo

    # 1. Decoding requests, oldest first.  Each must run; make room if needed.
    decoding, in_prompt = [], []
    for r in self.running:
      (decoding if r.is_decoding else in_prompt).append(r)
    decoding.sort(key=lambda r: r.arrival)
    if decoding and len(decoding) <= budget and self.cache.pages_short([(r.slot, 1) for r in decoding]) == 0:
      # The usual case, decided with one look at the pools: all of them fit, so each prefix does.
      for r in decoding:
        chosen.append((r.slot, 1))
        plan.entries.append(PlannedEntry(r, 1, True))
      budget -= len(decoding)
      decoding = []
    for r in decoding:
      if r.status is not Status.RUNNING:
        continue  # preempted below while making room for an older one
      if budget == 0:
        break
      while not fits(r.slot, 1):
        victim = self._youngest_running(exclude=r, chosen_slots={s for s, _ in chosen})
        if victim is None:
          break
        self._preempt(victim)
        plan.preempted.append(victim)
      if not fits(r.slot, 1):
        if not chosen:
          self._finish(r, "out_of_pages")
          plan.failed.append(r)
        continue
      chosen.append((r.slot, 1))
      plan.entries.append(PlannedEntry(r, 1, True))
      budget -= 1

    # 2. Prompt portions of live requests, oldest first.
    for r in sorted(in_prompt, key=lambda r: r.arrival):
      if r.status is not Status.RUNNING:
        continue  # preempted above
      if budget == 0:
        break
      n = largest_fitting(r.slot, min(r.remaining, budget))
      if n == 0:
        continue
      chosen.append((r.slot, n))
      plan.entries.append(PlannedEntry(r, n, n == r.remaining))
      budget -= n

    # 3. New requests, first come first served, while slots, budget and pages allow.
    # (Not in a step that had to take pages away from a live request.)
    while self.waiting and budget > 0 and self.cache.num_free_slots > 0 and not plan.preempted:
      r = self.waiting[0]
      slot = self.cache.acquire_slot(r.request_id)
      n = largest_fitting(slot, min(r.remaining, budget))
      if n == 0:
        self.cache.release_slot(slot)
        if not self.running and not chosen:
          # Nothing else holds pages, and still not one token fits.
          self.waiting.popleft()
          self._finish(r, "out_of_pages")
          plan.failed.append(r)
          continue
        break
      self.waiting.popleft()
      r.slot, r.status = slot, Status.RUNNING
      self.running.append(r)
      chosen.append((slot, n))
      plan.entries.append(PlannedEntry(r, n, n == r.remaining))
      budget -= n

    # A live request that alone cannot go on, with nothing else to wait for, cannot ever.
    if not plan.entries and self.running and not plan.preempted:
      r = min(self.running, key=lambda r: r.arrival)
      if len(self.running) == 1:
        self._finish(r, "out_of_pages")
        plan.failed.append(r)
      else:
        victim = self._youngest_running(exclude=r, chosen_slots=set())
        self._preempt(victim)
        plan.preempted.append(victim)
    return plan

  def _youngest_running(self, exclude: Request, chosen_slots: set[int]) -> Request | None:
    candidates = [r for r in self.running if r is not exclude and r.slot not in chosen_slots]
    return max(candidates, key=lambda r: r.arrival) if candidates else None

  def _preempt(self, r: Request) -> None:
    self.cache.release_slot(r.slot)
    self.running.remove(r)
    r.slot, r.num_cached, r.status = None, 0, Status.WAITING
    r.num_preemptions += 1
    self.waiting.appendleft(r)

  # ---- after the step -----------------------------------------------------------
  def commit(self, plan: StepPlan, sampled: dict[object, int],
             logprobs: dict[object, float] | None = None) -> list[Request]:
    """Records the step's progress and sampled tokens (and their log-probabilities, where the
    step computed them); returns requests that ended."""
    finished = []
    for e in plan.entries:
      r = e.request
      if r.status is not Status.RUNNING:
        continue  # cancelled while the step ran
      r.num_cached += e.num_tokens
      if not e.samples:
        continue
      token = int(sampled[r.request_id])
      r.tokens.append(token)
      if logprobs is not None and r.params.logprobs:
        r.logprobs.append(float(logprobs[r.request_id]))
      stops = r.params.stop_token_ids if r.params.stop_token_ids is not None else self.eos_ids
      if token in stops:
        reason = "eos"
      elif r.num_output >= r.params.max_decode_steps:
        reason = "max_decode_steps"
      elif len(r.tokens) >= self.max_seq_len:
        reason = "max_seq_len"
      else:
        continue
      self._finish(r, reason)
      finished.append(r)
    return finished

  def _finish(self, r: Request, reason: str) -> None:
    if r.status is Status.RUNNING:
      self.cache.release_slot(r.slot)
      self.running.remove(r)
    elif r in self.waiting:
      self.waiting.remove(r)
    r.slot = None
    r.status = Status.FINISHED
    r.finish_reason = reason
