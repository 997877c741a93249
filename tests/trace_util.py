"""Builds replay traces (four ways of cutting the same requests) and runs them.

A trace is a list of step objects in the replay tool's input format.  Every
builder asks for the logits of *every* fed token, so a run yields, per request,
the logits at all its positions, to be compared with the plain model's
whole-sequence logits.
"""

from __future__ import annotations

import io
import json
import os
import subprocess
import sys

import numpy as np

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(REPO, "bin", "trace_run")


def _entry(rid, tokens, start, n):
  return {"id": rid, "tokens": [int(t) for t in tokens[start:start + n]], "want": list(range(n))}


def whole(requests):
  """Each request alone, in one step."""
  return [{"step": i, "entries": [_entry(rid, toks, 0, len(toks))], "end": [rid]}
          for i, (rid, toks) in enumerate(requests.items())]


def prefill_then_decode(requests, tail=32):
  """All but the last `tail` tokens in one step, then the rest one by one."""
  steps = []
  for rid, toks in requests.items():
    head = max(len(toks) - tail, 1)
    cuts = [head] + [1] * (len(toks) - head)
    pos = 0
    for j, n in enumerate(cuts):
      steps.append({"step": len(steps), "entries": [_entry(rid, toks, pos, n)],
                    "end": [rid] if j == len(cuts) - 1 else []})
      pos += n
  return steps


def changing_portions(requests, sizes=(7, 2, 5, 3, 11, 2, 13, 4, 2, 9)):
  """Each request alone, in portions of changing size, down to two tokens."""
  steps = []
  for rid, toks in requests.items():
    pos, j = 0, 0
    while pos < len(toks):
      n = min(sizes[j % len(sizes)], len(toks) - pos)
      pos_after = pos + n
      steps.append({"step": len(steps), "entries": [_entry(rid, toks, pos, n)],
                    "end": [rid] if pos_after == len(toks) else []})
      pos, j = pos_after, j + 1
  return steps


def mixed(requests, seed=0, max_live=4, decode_after=0.5, portions=(2, 3, 5, 7, 9)):
  """Up to `max_live` requests live at once: portions of some beside single tokens of
  others, requests starting as others end (so pages are used again), a request
  sometimes left out of a step."""
  rng = np.random.default_rng(seed)
  waiting = list(requests.items())
  live = {}  # rid -> [tokens, position]
  steps = []
  while waiting or live:
    while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
      rid, toks = waiting.pop(0)
      live[rid] = [toks, 0]
    entries, ended = [], []
    for rid, (toks, pos) in list(live.items()):
      if len(live) > 1 and rng.random() < 0.2:
        continue  # left out of this step
      left = len(toks) - pos
      if pos >= decode_after * len(toks):
        n = 1
      else:
        n = min(int(rng.choice(portions)), left)
      entries.append(_entry(rid, toks, pos, n))
      live[rid][1] = pos + n
      if pos + n == len(toks):
        ended.append(rid)
        del live[rid]
    if entries:
      steps.append({"step": len(steps), "entries": entries, "end": ended})
  return steps


def tokens_needed(steps, page=64):
  """Most tokens live requests hold at any time, each rounded up to a page."""
  held, worst = {}, 0
  for s in steps:
    for e in s["entries"]:
      held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
    worst = max(worst, sum(-(-n // page) * page for n in held.values()))
    for rid in s["end"]:
      held.pop(rid, None)
  return worst


def collect(steps, out_dir, vocab):
  """Reads the <step>.f32 files back: {request id: {position: logits row}}."""
  got, pos = {}, {}
  for s in steps:
    rows = sum(len(e["want"]) for e in s["entries"])
    if rows == 0:
      continue
    arr = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4")
    assert arr.size == rows * vocab, (s["step"], arr.size, rows, vocab)
    arr = arr.reshape(rows, vocab)
    r = 0
    for e in s["entries"]:
      start = pos.get(e["id"], 0)
      for w in e["want"]:
        got.setdefault(e["id"], {})[start + w] = arr[r]
        r += 1
      pos[e["id"]] = start + len(e["tokens"])
  # positions advance also in steps that want nothing
  return got


def run_in_process(engine, steps, out_dir):
  """Drives `simply_b200.engine.replay.replay` directly (CPU tests with the reference kernel table)."""
  from simply_b200.engine.replay import replay

  lines = io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n")
  sink = io.StringIO()
  n = replay(engine, lines, out_dir, sink)
  assert sink.getvalue().split() == [w for s in steps for w in ("done", str(s["step"]))]
  return n


def run_tool(model_dir, dtype, steps, out_dir, max_tokens, extra=(), timeout=600):
  """Runs bin/trace_run as a user would: one line in, wait for `done <step>`, next line."""
  cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
         "--max-tokens", str(max_tokens), *extra]
  p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                       text=True)
  try:
    for s in steps:
      p.stdin.write(json.dumps(s) + "\n")
      p.stdin.flush()
      while True:
        line = p.stdout.readline()
        if not line:
          raise AssertionError(f"trace_run ended early at step {s['step']}:\n{p.stderr.read()}")
        if line.strip() == f"done {s['step']}":
          break
    p.stdin.close()
    rc = p.wait(timeout=timeout)
    err = p.stderr.read()
    assert rc == 0, f"trace_run exited with {rc}:\n{err}"
  finally:
    if p.poll() is None:
      p.kill()
