"""One step's batch: which requests bring which tokens, and the metadata kernels read.

A step is a list of entries `(slot, tokens, want)`: the next tokens of a live
request (a portion of its prompt, or one decoded token) and the places among
them whose logits are wanted.  The tokens of all entries are packed into one
ragged batch; nothing is padded.

The reference packs the same information into a padded `tokens[1, capacity]`
row with `segment_ids` (slot + 1, 0 for padding) and `segment_positions`
(simply/utils/ragged_paged_attention.py:1992-2010) plus per-layer `kv_lens`
and `page_indices`; here every array is exact-size and block tables exist once
per page group, not per layer.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Sequence

import numpy as np
import torch


@dataclasses.dataclass(frozen=True)
class StepEntry:
  slot: int
  tokens: Sequence[int]
  want: Sequence[int] = ()  # indices into `tokens`


@dataclasses.dataclass
class StepContext:
  """Everything a part may read during one step.  Device tensors unless noted.

  Sequences are the entries of the step, in order; token t belongs to sequence
  `token_seq[t]` and sits at position `positions[t]` of its request.  The new
  tokens of sequence b are rows cu_q[b] .. cu_q[b+1]-1 and continue the
  `q_start[b]` tokens that are already cached.
  """

  ops: Any
  num_tokens: int  # host int
  num_seqs: int  # host int
  token_ids: torch.Tensor  # i32 [T]
  positions: torch.Tensor  # i32 [T]
  token_seq: torch.Tensor  # i32 [T]
  cu_q: torch.Tensor  # i32 [B+1]
  q_start: torch.Tensor  # i32 [B]
  slots: torch.Tensor  # i32 [B]
  block_tables: list[torch.Tensor]  # per page group: i32 [B, max_pages_per_seq]
  logit_rows: torch.Tensor  # i32 [R] rows (tokens) whose logits are wanted
  # Host-side facts for launch decisions.
  max_q_len: int
  max_kv_len: int
  page_size: int
  # Host copies (NumPy) for parts that are written in plain torch (toy parts in tests).
  host: dict[str, np.ndarray] = dataclasses.field(default_factory=dict)
  # Scratch shared by the parts of one step, e.g. rotation tables keyed by their parameters.
  memo: dict[Any, Any] = dataclasses.field(default_factory=dict)
  # True when every cached key and value below q_start was written by an earlier step (the engine
  # sets it): decode attention may then fetch them while the kernel before it still runs.
  older_keys_settled: bool = False


def pack_step(entries: Sequence[StepEntry], lengths_before: Sequence[int],
              group_tables: Sequence[np.ndarray], page_size: int, ops: Any,
              device: torch.device | str, token_arrays: Sequence[np.ndarray] | None = None) -> StepContext:
  """Builds the step's metadata on the host and moves it to the device in one copy.

  lengths_before[i]: tokens already cached for entry i.  group_tables[g]: the
  page group's full block table `[max_slots, max_pages]` (host); only the rows of
  the step's slots are sent.
  """
  num_seqs = len(entries)
  q_lens = np.array([len(e.tokens) for e in entries], dtype=np.int64)
  if num_seqs == 0 or (q_lens <= 0).any():
    raise ValueError("a step needs at least one entry and every entry at least one token")
  cu_q = np.zeros(num_seqs + 1, dtype=np.int32)
  np.cumsum(q_lens, out=cu_q[1:])
  num_tokens = int(cu_q[-1])
  q_start = np.asarray(lengths_before, dtype=np.int32)
  if token_arrays is None:  # (the caller may have made arrays of the tokens already)
    token_arrays = [np.asarray(e.tokens) for e in entries]
  token_ids = np.concatenate(token_arrays).astype(np.int32, copy=False)
  token_seq = np.repeat(np.arange(num_seqs, dtype=np.int32), q_lens)
  positions = (np.arange(num_tokens, dtype=np.int32) - cu_q[:-1][token_seq] + q_start[token_seq])
  slots = np.array([e.slot for e in entries], dtype=np.int32)
  rows = []
  for i, e in enumerate(entries):
    for w in e.want:
      if not 0 <= w < len(e.tokens):
        raise ValueError(f"entry {i}: wanted place {w} is outside its {len(e.tokens)} tokens")
      rows.append(int(cu_q[i]) + int(w))
  logit_rows = np.asarray(rows, dtype=np.int32)
  tables = [np.ascontiguousarray(t[slots]) for t in group_tables]

  # One host buffer, one copy; the device tensors are views of it.
  parts = [token_ids, positions.astype(np.int32), token_seq, cu_q, q_start, slots, logit_rows]
  parts += [t.reshape(-1) for t in tables]
  sizes = [p.size for p in parts]
  flat = np.concatenate(parts).astype(np.int32, copy=False)
  host = torch.from_numpy(flat)
  dev = torch.device(device)
  if dev.type == "cuda":
    host = host.pin_memory()
  buf = host.to(dev, non_blocking=True)
  views = list(torch.split(buf, sizes))
  n_fixed = 7
  block_tables = [v.view(num_seqs, t.shape[1]) for v, t in zip(views[n_fixed:], tables)]
  return StepContext(
      ops=ops, num_tokens=num_tokens, num_seqs=num_seqs,
      token_ids=views[0], positions=views[1], token_seq=views[2], cu_q=views[3],
      q_start=views[4], slots=views[5], block_tables=block_tables, logit_rows=views[6],
      max_q_len=int(q_lens.max()), max_kv_len=int((q_start + q_lens).max()),
      page_size=page_size,
      host={"cu_q": cu_q, "q_start": q_start, "slots": slots, "positions": positions,
            "token_seq": token_seq, "logit_rows": logit_rows})
