"""Builds a paged-cache scenario for kernel tests: slots with history, a step on top of it.

`make_scenario` uses the real cache manager and `pack_step`, so block tables,
released window pages and page reuse look exactly as in the engine.  Cache
storage is random where a request holds tokens and NaN everywhere else (free
pages, released pages, the unwritten tail of a last page), so any read outside
what a request holds poisons the result.
"""

from __future__ import annotations

import dataclasses

import numpy as np
import torch

from simply_b200.cache import CacheManager, PagedKVNeed
from simply_b200.engine.batch import StepEntry, pack_step


@dataclasses.dataclass
class Scenario:
  manager: CacheManager
  ctx: object
  cache: object  # PagedCache
  storage: torch.Tensor
  block_table: torch.Tensor
  seqs: list  # (slot, q_start, q_len)


def make_scenario(seqs, *, num_kv_heads, head_dim, window, page_size, dtype, device, ops, seed=0,
                  extra_pages=3, churn=True):
  """seqs: list of (history tokens, new tokens)."""
  rng = np.random.default_rng(seed)
  max_len = max(h + n for h, n in seqs) + page_size
  total_tokens = sum(-(-(h + n) // page_size) * page_size for h, n in seqs) + extra_pages * page_size
  mgr = CacheManager({"c": PagedKVNeed(num_kv_heads, head_dim, window)}, page_size=page_size,
                     max_slots=len(seqs) + 1, max_seq_len=max_len, max_cache_tokens=total_tokens,
                     dtype=dtype, device=device)
  if churn:
    # Take and give back a few pages first so that page ids are not handed out in order.
    s = mgr.acquire_slot("churn")
    mgr.extend([(s, min(extra_pages * page_size, max_len))])
    mgr.release_slot(s)
  slots = []
  for i, (hist, _) in enumerate(seqs):
    slot = mgr.acquire_slot(i)
    slots.append(slot)
    done = 0
    while done < hist:  # history arrives in uneven portions, as prompts do
      n = int(min(hist - done, rng.integers(1, 3 * page_size)))
      mgr.extend([(slot, n)])
      done += n
  entries = [StepEntry(slot, [0] * n, ()) for slot, (_, n) in zip(slots, seqs)]
  lengths = [mgr.length(s) for s in slots]
  mgr.extend([(e.slot, len(e.tokens)) for e in entries])
  mgr.check_invariants()
  ctx = pack_step(entries, lengths, [g.tables for g in mgr.groups], page_size, ops, device)
  cache = mgr.paged["c"]
  st = cache.storage
  st.fill_(float("nan"))
  g = mgr.groups[0]
  gen = torch.Generator(device="cpu")
  gen.manual_seed(seed)
  for slot, (hist, n) in zip(slots, seqs):
    length = hist + n
    first = int(g.first_page[slot])
    for pi in range(first, int(g.end_page[slot])):
      page = int(g.tables[slot, pi])
      valid = min(page_size, length - pi * page_size)
      vals = torch.randn(2, num_kv_heads, valid, head_dim, generator=gen)
      st[page, :, :, :valid, :] = vals.to(dtype).to(device)
  return Scenario(mgr, ctx, cache, st, ctx.block_tables[0], list(zip(slots, lengths, [n for _, n in seqs])))
