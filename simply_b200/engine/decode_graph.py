"""Decode steps replayed from CUDA graphs, several in a row without the host in between.

A step in which every live request brings exactly one token always launches the
same kernels; only a few integers change.  The runner keeps those integers in one
static device buffer, captures the whole step (model, sampling, and a tiny kernel
that turns the sampled tokens into the next step's inputs) in a CUDA graph per
(batch size, length bucket), and replays it.  A burst of n replays needs one
host-to-device copy before and one device-to-host copy after, which is the
reference's on-device decode loop (`continue_decode` with `intermediate_steps`,
simply/utils/ragged_paged_attention.py:2064-2102, simply/serving/common_flags.py:84-86)
without a tracing compiler.

The pages for all n tokens of every request are taken before the burst, so block
tables do not change inside it.  What a mixer prepares on the host per step (the
split-key attention work lists) it hands over as plans (`Mixer.graph_plans`): the
runner gives each plan a piece of the static buffer and lets it refill that piece
before a burst; the lists cover the keys of the whole burst, and chunks with nothing
visible at a given step come out empty.

Which models run this way is the parts' own statement (`graph_safe`), not a list kept
here: any registered part that keeps to device tensors and `ctx.memo` takes part.
"""

from __future__ import annotations

import ctypes
import dataclasses
import gc
from typing import Any, Sequence

import numpy as np
import torch

from simply_b200.engine.batch import StepContext
from simply_b200.kernels.ops import KernelError


def graphable(model: Any) -> bool:
  """Graphs are used when every part says that its step may be captured (`Part.graph_safe`):
  a part that reads host-side metadata, which a replay does not refresh, or waits for the
  device, which a capture forbids, leaves the flag at its default and the model runs eagerly."""
  return bool(model.graph_safe())


@dataclasses.dataclass
class _Graph:
  graph: torch.cuda.CUDAGraph
  meta: torch.Tensor  # static int32 buffer on the device
  host: torch.Tensor  # pinned mirror
  views: dict[str, tuple[int, int]]  # name -> (offset, size) in words
  plans: dict[tuple, dict]
  sampled: torch.Tensor
  history: torch.Tensor
  host_history: torch.Tensor  # pinned
  step_fn: Any
  captured: bool
  batch: int
  bucket: int
  launches: int
  logits_history: torch.Tensor | None = None  # [MAX_BURST, batch, vocab] when logits are kept
  logprob_history: torch.Tensor | None = None  # [MAX_BURST, batch] when the graph computes log-probabilities
  resume: dict | None = None  # what the device holds after the last burst (see DecodeRunner.run)
  graph_exec: Any = None  # the instantiated graph's handle and the buffers' addresses, for the native launch
  pointers: tuple = ()


class DecodeRunner:

  MAX_BURST = 64

  def __init__(self, engine: Any):
    self.engine = engine
    self.ops = engine.ops
    self.graphs: dict[tuple[int, int, bool], _Graph] = {}
    self.last_logprobs: np.ndarray | None = None  # [steps, live] after a burst run with logprobs
    # True keeps the float32 logits of every step of a burst on the device (`last_logits` after
    # `run`): tests compare the rows a replay produced with a plain model's.  Set before the
    # first burst; costs MAX_BURST * batch * vocab floats per graph.
    self.keep_logits = False
    self.last_logits: torch.Tensor | None = None
    self.stream = torch.cuda.Stream(device=engine.device)
    self._stream_ptr = ctypes.c_void_p(self.stream.cuda_stream)
    self.pool = torch.cuda.graph_pool_handle()
    self.bursts = 0  # bursts run so far, and how many of them went on from the device's own state
    self.resumed_bursts = 0
    self.h2d_bytes = 0  # bytes copied to and from the device by `run` so far
    self.d2h_bytes = 0

  def batch_bucket(self, live: int) -> int:
    """The batch size of the graph that serves `live` requests: 1, 2, 4, 8, then steps of 8 up
    to 32, of 16 up to 64, of 32 beyond (the weight-streaming products cost the same for 1 to 8
    and for 9 to 16 rows; attention and the output layer grow with the rows), never more than
    the engine's slots unless `live` itself is."""
    if live <= 8:
      size = 1 << (live - 1).bit_length()
    elif live <= 32:
      size = -(-live // 8) * 8
    elif live <= 64:
      size = -(-live // 16) * 16
    else:
      size = -(-live // 32) * 32
    return max(live, min(size, self.engine.cache.max_slots))

  # ---- layout of the static buffer -----------------------------------------------
  def _plans(self, batch: int, bucket: int) -> list:
    """The plans of all mixers for this graph, one per memo key (layers of one kind share theirs)."""
    plans: dict[Any, Any] = {}
    for block in self.engine.model.blocks.values():
      for plan in block.mixer.graph_plans(self.ops, batch, bucket, self.MAX_BURST, self.engine.cache.page_size):
        plans.setdefault(plan.key, plan)
    return list(plans.values())

  def _layout(self, batch: int, bucket: int, plans: list) -> tuple[dict, int]:
    cache = self.engine.cache
    views, off = {}, 0

    def take(name, size):
      nonlocal off
      views[name] = (off, size)
      off += size

    for name in ("token_ids", "positions", "token_seq", "q_start", "slots", "logit_rows"):
      take(name, batch)
    take("cu_q", batch + 1)
    take("step_counter", 1)
    take("sample_params", batch * 6)
    for gi, g in enumerate(cache.groups):
      take(f"table{gi}", batch * g.max_pages_per_seq)
    for i, plan in enumerate(plans):
      take(f"plan{i}", plan.words)
    return views, off

  def _prepare(self, batch: int, bucket: int, logprobs: bool = False) -> _Graph:
    """Static buffers and the step closure for one (batch, bucket); nothing runs yet.  With
    `logprobs` the step also records the log-probability of every sampled token."""
    eng, ops = self.engine, self.ops
    plan_list = self._plans(batch, bucket)
    views, words = self._layout(batch, bucket, plan_list)
    meta = torch.zeros(words, dtype=torch.int32, device=eng.device)
    host = torch.zeros(words, dtype=torch.int32).pin_memory()

    def view(name):
      o, n = views[name]
      return meta[o:o + n]

    block_tables = [view(f"table{gi}").view(batch, g.max_pages_per_seq)
                    for gi, g in enumerate(eng.cache.groups)]
    ctx = StepContext(
        ops=ops, num_tokens=batch, num_seqs=batch, token_ids=view("token_ids"), positions=view("positions"),
        token_seq=view("token_seq"), cu_q=view("cu_q"), q_start=view("q_start"), slots=view("slots"),
        block_tables=block_tables, logit_rows=view("logit_rows"), max_q_len=1, max_kv_len=bucket,
        page_size=eng.cache.page_size, older_keys_settled=True)
    bound = {plan.key: plan.bind(view(f"plan{i}")) for i, plan in enumerate(plan_list)}
    plans = {f"plan{i}": plan for i, plan in enumerate(plan_list)}
    sampled = torch.zeros(batch, dtype=torch.int32, device=eng.device)
    history = torch.zeros(self.MAX_BURST, batch, dtype=torch.int32, device=eng.device)
    host_history = torch.zeros(self.MAX_BURST, batch, dtype=torch.int32).pin_memory()
    logits_history = None
    if self.keep_logits:
      logits_history = torch.zeros(self.MAX_BURST, batch, eng.model.spec.vocab_size, dtype=torch.float32,
                                   device=eng.device)

    logprob_history = None
    if logprobs:
      logprob_history = torch.zeros(self.MAX_BURST, batch, dtype=torch.float32, device=eng.device)

    def one_step():
      ctx.memo = dict(bound)
      logits = eng.model.forward(ctx, eng.caches)
      if logits_history is not None:
        ops.keep_logits(logits, logits_history, view("step_counter"))
      ops.sample_device(logits, view("sample_params").view(batch, 6), sampled, logprobs_out=logprob_history,
                        step_counter=view("step_counter") if logprobs else None)
      ops.decode_advance(sampled, view("token_ids"), view("positions"), view("q_start"),
                         view("sample_params"), history, view("step_counter"))

    g = _Graph(torch.cuda.CUDAGraph(), meta, host, views, plans, sampled, history, host_history, one_step,
               False, batch, bucket, 0, logits_history, logprob_history)
    self._fill_constants(g)
    return g

  def _first_step_and_capture(self, g: _Graph) -> None:
    """Runs the burst's first step eagerly on the capture stream (this also sets up library
    handles and kernel attributes), then records the same step into the graph.  Recording
    executes nothing, so the state stays where the eager step left it."""
    current = torch.cuda.current_stream(self.engine.device)
    self.stream.wait_stream(current)
    with torch.cuda.stream(self.stream):
      g.step_fn()
      self.stream.synchronize()
      before = self.ops.launches
      # No garbage collection while the stream captures: a collected object that frees device
      # resources (an older graph, say) would make a call that a capture forbids and spoil it.
      gc_was_on = gc.isenabled()
      gc.disable()
      try:
        # (Not through torch.cuda.graph(): it empties the allocator's caches first, which costs
        # more than the capture.  All graphs share one pool: they never run at the same time.)
        g.graph.capture_begin(pool=self.pool)
        try:
          g.step_fn()
        finally:
          g.graph.capture_end()
      finally:
        if gc_was_on:
          gc.enable()
      g.launches = self.ops.launches - before
    self.stream.synchronize()
    g.captured = True

  def _fill_constants(self, g: _Graph) -> None:
    b = g.batch
    h = g.host.numpy()

    def put(name, values):
      o, n = g.views[name]
      h[o:o + n] = np.asarray(values, dtype=np.int32).reshape(-1)

    put("token_seq", np.arange(b))
    put("logit_rows", np.arange(b))
    put("cu_q", np.arange(b + 1))
    put("step_counter", [0])

  # ---- running -----------------------------------------------------------------------
  def _chunk_ranges(self, g, lengths: np.ndarray, steps: int) -> list:
    return [plan.ranges(lengths, steps) for plan in g.plans.values()]

  @staticmethod
  def _same_ranges(a: list, b: list) -> bool:
    return all(len(x) == len(y) and all(np.array_equal(p, q) for p, q in zip(x, y)) for x, y in zip(a, b))

  def run(self, slots: Sequence[int], last_tokens: Sequence[int], sample_params: np.ndarray,
          steps: int, logprobs: bool = False) -> np.ndarray:
    """Decodes `steps` tokens for every slot; returns the sampled tokens [steps, batch].  With
    `logprobs`, `last_logprobs` [steps, batch] then holds the tokens' log-probabilities.

    `last_tokens[i]` is the not yet cached last token of slot i; `sample_params` is the
    [batch, 6] word table of csrc/sampling.cu with the position of the first token to sample.
    """
    eng = self.engine
    cache = eng.cache
    live = len(slots)
    if not 1 <= steps <= self.MAX_BURST:
      raise ValueError(f"a decode burst has 1..{self.MAX_BURST} steps, got {steps}")
    lengths = cache.lengths[np.asarray(slots, dtype=np.int64)]
    cache.extend([(s, steps) for s in slots])
    # Graphs exist for a few batch sizes only (a capture costs tens of milliseconds, and a batch
    # that shrinks as requests end would need one per size).  The rows up to the next such size
    # repeat the last request: they compute what it computes, store the same keys and values to
    # the same places, and their tokens are dropped.
    batch = self.batch_bucket(live)
    if batch > live:
      pad = batch - live
      slots = list(slots) + [slots[-1]] * pad
      last_tokens = list(last_tokens) + [last_tokens[-1]] * pad
      sample_params = np.asarray(sample_params, dtype=np.int32).reshape(live, 6)
      sample_params = np.concatenate([sample_params, np.repeat(sample_params[-1:], pad, axis=0)])
      lengths = np.concatenate([lengths, np.repeat(lengths[-1:], pad)])
    bucket = 1024
    while bucket < int(lengths.max()) + steps:
      bucket *= 2
    key = (batch, bucket, bool(logprobs))
    g = self.graphs.get(key)
    if g is None:
      g = self.graphs[key] = self._prepare(batch, bucket, bool(logprobs))
    # What the device would need to be told.  If it is exactly what the last burst of this graph
    # left behind (same requests one step on, no page taken or given back, the same key chunks),
    # the device's own copy, advanced by the graph itself, is already right: only the tokens are
    # uploaded.
    slots_t = tuple(int(s) for s in slots)
    last_tokens = np.asarray(last_tokens, dtype=np.int32)
    sample_params = np.asarray(sample_params, dtype=np.int32).reshape(batch, 6)
    version = cache.tables_version()
    r = g.resume
    follows = (
        r is not None and g.captured and r["slots"] == slots_t and r["version"] == version
        and r["counter"] + steps <= self.MAX_BURST and np.array_equal(r["lengths"], lengths)
        and np.array_equal(r["params"], sample_params))
    if follows and r["next_steps"] == steps:
      # The last burst worked out, while the device ran, what a burst like itself would need next.
      ranges, resumed = r["next_ranges"], r["next_ranges_same"]
    else:
      ranges = self._chunk_ranges(g, lengths, steps)
      resumed = follows and self._same_ranges(r["ranges"], ranges)
    first_row = r["counter"] if resumed else 0
    self.bursts += 1
    self.resumed_bursts += bool(resumed)
    h = g.host.numpy()

    def put(name, values):
      o, n = g.views[name]
      h[o:o + n] = np.asarray(values, dtype=np.int32).reshape(-1)

    put("token_ids", last_tokens)  # the host's tokens go to the device in either case
    if not resumed:
      put("positions", lengths)
      put("q_start", lengths)
      put("slots", slots)
      put("step_counter", [0])
      put("sample_params", sample_params)
      for gi, grp in enumerate(cache.groups):
        put(f"table{gi}", grp.tables[np.asarray(slots)])
      for name, plan in g.plans.items():
        o, n = g.views[name]
        plan.fill(h[o:o + n], lengths, steps)
    # Copy, replays and read-back run on the runner's own stream, the one the graph was captured
    # on, issued by one native call.  (A burst that goes on from the last one needs no order with
    # the engine's stream: nothing ran there for these requests since, or their lengths would differ.)
    if not resumed:
      self.stream.wait_stream(torch.cuda.current_stream(eng.device))
    replays = steps
    o, n = g.views["token_ids"] if resumed else (0, g.meta.numel())
    if not g.captured:
      with torch.cuda.stream(self.stream):
        g.meta.copy_(g.host, non_blocking=True)
        self._first_step_and_capture(g)
      g.graph_exec = ctypes.c_void_p(g.graph.raw_cuda_graph_exec())
      g.pointers = (g.meta.data_ptr(), g.host.data_ptr(), g.history.data_ptr(), g.host_history.data_ptr())
      replays -= 1
      self.h2d_bytes += 4 * n
      n = 0  # already there
    meta_p, host_p, history_p, host_history_p = g.pointers
    row_bytes = 4 * batch
    rows = slice(first_row, first_row + steps)
    rc = self.ops.lib.sb_graph_burst(
        g.graph_exec, ctypes.c_void_p(meta_p + 4 * o), ctypes.c_void_p(host_p + 4 * o), 4 * n, replays,
        ctypes.c_void_p(host_history_p + first_row * row_bytes), ctypes.c_void_p(history_p + first_row * row_bytes),
        steps * row_bytes, self._stream_ptr)
    if rc != 0:
      raise KernelError(f"decode burst: CUDA error {rc}")
    self.h2d_bytes += 4 * n
    self.d2h_bytes += steps * row_bytes
    # While the device works: the state it will be in, as the next burst would have to describe
    # it, and whether a burst of the same length could go on from it.
    next_params = sample_params.copy()
    next_params[:, 5] += steps
    next_lengths = lengths + steps
    next_ranges = self._chunk_ranges(g, next_lengths, steps)
    g.resume = dict(slots=slots_t, version=version, counter=first_row + steps, lengths=next_lengths,
                    params=next_params, ranges=ranges, next_steps=steps, next_ranges=next_ranges,
                    next_ranges_same=self._same_ranges(ranges, next_ranges))
    rc = self.ops.lib.sb_stream_wait(self._stream_ptr)
    if rc != 0:
      raise KernelError(f"decode burst: CUDA error {rc}")
    out = g.host_history[rows].numpy()[:, :live].copy()
    if g.logits_history is not None:
      self.last_logits = g.logits_history[rows, :live].clone()
    if g.logprob_history is not None:
      self.last_logprobs = g.logprob_history[rows, :live].cpu().numpy()
    self.ops.launches += g.launches * replays
    eng.num_steps += steps
    return out
