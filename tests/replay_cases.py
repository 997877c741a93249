"""The requests and traces the replay tests use, shared by the CPU and GPU variants."""

import numpy as np

from tests import trace_util
from tests.tolerances import assert_logits_close, first_bad_position

# Lengths beyond the windows (8 and 16) and beyond one 64-token page.
LENGTHS = {"a": (70, 45, 90, 33, 131), "b": (66, 40, 23, 150, 77)}


def make_requests(which, vocab, seed=1):
  rng = np.random.default_rng(seed)
  return {f"r{i}": rng.integers(0, vocab, n).tolist() for i, n in enumerate(LENGTHS[which])}


MODES = {
    "whole": trace_util.whole,
    "tail": trace_util.prefill_then_decode,
    "portions": trace_util.changing_portions,
    "mixed": trace_util.mixed,
}


def combined_trace(requests, modes=("whole", "tail", "portions", "mixed")):
  """The four ways one after the other in a single trace; request ids carry the mode."""
  steps = []
  for mode in modes:
    renamed = {f"{mode}:{rid}": toks for rid, toks in requests.items()}
    for s in MODES[mode](renamed):
      s = dict(s, step=len(steps))
      steps.append(s)
  return steps


def compare(got, requests, expected, dtype):
  """got: {"mode:rid": {pos: row}}; expected: {rid: [T, V]}."""
  assert got, "no logits came back"
  for key, rows in sorted(got.items()):
    rid = key.split(":")[1]
    want = expected[rid]
    assert sorted(rows) == list(range(len(requests[rid]))), f"{key}: positions missing"
    bad = first_bad_position(rows, want, dtype)
    assert bad is None, (
        f"{key}: first wrong position {bad} of {len(want)} "
        f"(max diff {np.abs(rows[bad] - want[bad]).max():.3e}, scale {np.abs(want).max():.3e})")
    assert_logits_close(np.stack([rows[p] for p in sorted(rows)]), want, dtype, key)
