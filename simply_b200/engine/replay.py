"""Trace replay: feeds given token ids through the engine step by step and writes logits.

It samples nothing and owns no model code: every step goes through
`Engine.step_raw`, the step function that generation uses, with the same cache
manager and kernels.

Input, one JSON object per line on standard input:
  {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries`: per request its next tokens and the places among them whose logits
are wanted; all entries of a step form one batch.  `end`: requests that are
finished after this step; their slot and pages are given back.  For a step that
wants something, `<out>/<step>.f32` holds the logits `[wanted, vocab]` as
little-endian float32 in the order of the entries and of `want`.  After every
step the line `done <step>` is printed and flushed.

The reference has no such tool; its nearest relatives are test helpers
(simply/utils/ragged_paged_attention_test.py:36-60, simply/model_lib_test.py:597-618).
"""

from __future__ import annotations

import json
import os
import sys
from typing import IO

import numpy as np

from simply_b200.config import EngineConfig
from simply_b200.engine.batch import StepEntry
from simply_b200.engine.engine import Engine

def replay(engine: Engine, lines: IO[str], out_dir: str, out: IO[str] = sys.stdout,
           from_graph: bool = False) -> int:
  os.makedirs(out_dir, exist_ok=True)
  slots: dict[object, int] = {}
  steps = 0
  for line in lines:
    line = line.strip()
    if not line:
      continue
    msg = json.loads(line)
    step = msg["step"]
    entries = []
    for e in msg.get("entries", []):
      rid = e["id"]
      if rid not in slots:
        slots[rid] = engine.open_request(rid)
      entries.append(StepEntry(slots[rid], [int(t) for t in e["tokens"]],
                               [int(w) for w in e.get("want", [])]))
    if entries:
      logits = engine.step_raw(entries, from_graph=from_graph)
      if logits is not None:
        arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
        arr.tofile(os.path.join(out_dir, f"{step}.f32"))
      engine.ops.check_errors()
    for rid in msg.get("end", []):
      if rid in slots:
        engine.close_request(slots.pop(rid))
    steps += 1
    print(f"done {step}", file=out, flush=True)
  return steps


def engine_for_replay(model_dir: str, dtype: str, max_tokens: int, page_size: int = 64,
                      poison_freed_pages: bool = False, ops=None, max_live: int = 4,
                      cuda_graphs: bool = False) -> Engine:
  """An engine whose cache pool holds `max_tokens` tokens (rounded up to whole pages) and that
  serves up to `max_live` requests at a time.  With `cuda_graphs`, steps in which every request
  brings one token are replayed from the decode graphs that generation uses."""
  from simply_b200.config import load_config

  max_context = load_config(model_dir).model_spec().max_context
  pages = -(-max_tokens // page_size)
  ec = EngineConfig(
      activation_dtype=dtype, page_size=page_size, batch_size=max_live,
      max_seq_len=max_context, max_cache_tokens=pages * page_size,
      max_window_cache_tokens=-1,  # a trace may bring a portion of any length in one step
      poison_freed_pages=poison_freed_pages, use_cuda_graphs=cuda_graphs)
  engine = Engine.from_folder(model_dir, ec, ops=ops)
  if engine._decode_runner is not None:
    engine._decode_runner.keep_logits = True
  return engine


def main(argv=None) -> int:
  import argparse

  ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
  ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
  ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
  ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
  ap.add_argument("--max-tokens", type=int, required=True,
                  help="most tokens live requests hold at any time (each rounded up to a page)")
  ap.add_argument("--page-size", type=int, default=64, help="tokens per cache page (default 64)")
  ap.add_argument("--poison-freed-pages", action="store_true",
                  help="fill pages that are given back with NaN (shows reads of pages not held)")
  ap.add_argument("--max-live", type=int, default=4, help="requests that may be live at a time (default 4)")
  ap.add_argument("--cuda-graphs", action="store_true",
                  help="replay steps that bring one token per request from the decode graphs of generation")
  args = ap.parse_args(argv)
  engine = engine_for_replay(args.model, args.dtype, args.max_tokens, args.page_size,
                             args.poison_freed_pages, max_live=args.max_live, cuda_graphs=args.cuda_graphs)
  replay(engine, sys.stdin, args.out, from_graph=args.cuda_graphs)
  return 0
