"""Benchmark: Gemma 2 2B shape, random bfloat16 weights, one B200.

  python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 with every
sequence ending at the full context (8,192 cached tokens), timed on the device over K
decode steps that run back to back from CUDA graphs; the figure is the median of five
such bursts of K steps, each bracketed by events of its own (the last burst ends at the
full context, the first 4 K tokens before it).  `e2e` is the same through the
public entry point (`Engine.add_request` / `Engine.step`), host tokens in and out, one
host round trip per step.  `prefill` is one 2,048-token prompt in one step (the median of five
such steps, each after a quarter of a second of rest: a prompt arrives on its own, and a GPU that
has just run tens of milliseconds at full power is held back by its power limit); `points`
holds decode at batch 1 and 64 (other presets: the batches their configuration names), at
batch 8 with contexts of 1,024 and 4,096, prompts of 4,096 and 8,192 tokens in one step, and a serving-like run through `Engine.generate` (128
requests over 64 slots, prompts of about 512 and outputs of about 128 tokens); `roofline`
relates the decode step's bytes (every weight once, plus the cache of the live requests) to the
measured copy bandwidth; `kernels` gives the dominant kernels' own fractions, each timed alone
over all layers' weights or caches: the weight-streaming products and the split-key attention of
a decode step (of the copy bandwidth), the gate-up product with its activation of a 2,048-token
prefill (of the matrix-product peak).

A step reads 5.2 GB of weights and 0.65 GB of cache per sequence, far more than the
126 MB L2, so no L2 flush is needed between timed steps ("inputs larger than L2").
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def _find_number(tree, key):
  """The number stored under `key` anywhere in a JSON tree (directly, or as {"value": number})."""
  if isinstance(tree, dict):
    if key in tree:
      v = tree[key]
      if isinstance(v, dict):
        v = v.get("value")
      if isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0:
        return float(v)
    for child in tree.values():
      found = _find_number(child, key)
      if found is not None:
        return found
  elif isinstance(tree, list):
    for child in tree:
      found = _find_number(child, key)
      if found is not None:
        return found
  return None


def load_peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  if os.path.isfile(path):
    try:
      with open(path) as f:
        d = json.load(f)
      peaks = {}
      for k in FALLBACK_PEAKS:
        v = _find_number(d, k)
        if v is not None:
          peaks[k] = v
      if "hbm_gbs" in peaks and "bf16_tflops" in peaks:
        peaks.setdefault("bf16_tflops_sustained", peaks["bf16_tflops"])
        return peaks, "measured"
    except (ValueError, KeyError, TypeError):
      pass
  return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
  """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

  QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
           "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

  def __init__(self):
    self.rows = []
    self.proc = None
    self.thread = None

  def start(self):
    try:
      self.proc = subprocess.Popen(
          ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
          stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    except OSError:
      return
    self.thread = threading.Thread(target=self._read, daemon=True)
    self.thread.start()

  def _read(self):
    for line in self.proc.stdout:
      parts = [p.strip() for p in line.split(",")]
      if len(parts) == 6:
        self.rows.append(parts)

  def stop(self):
    if self.proc is None:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    self.proc.terminate()
    try:
      self.proc.wait(timeout=5)
    except subprocess.TimeoutExpired:
      self.proc.kill()
    clocks = sorted(int(r[0]) for r in self.rows if r[0].isdigit())
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
    return {
        "sm_mhz": clocks[len(clocks) // 2] if clocks else None,
        "sm_max_mhz": max((int(r[1]) for r in self.rows if r[1].isdigit()), default=None),
        "reasons": reasons,
        "samples": len(self.rows),
    }


def model_numbers(cfg, layers):
  """Bytes and FLOPs of the model from its config (layers may be fewer than the config's)."""
  d, f, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
  hq, hkv, dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
  per_layer = d * (hq + 2 * hkv) * dh + hq * dh * d + 3 * d * f + 4 * d
  params = layers * per_layer + v * d + d
  return {"per_layer_params": per_layer, "params": params, "weight_bytes": 2 * params,
          "kv_bytes_per_token_layer": 2 * hkv * dh * 2}


def decode_bytes(cfg, layers, batch, context):
  n = model_numbers(cfg, layers)
  types = cfg.resolved_layer_types()[:layers]
  kv = 0
  for t in types:
    seen = min(context, cfg.sliding_window) if t == "sliding_attention" else context
    kv += seen * n["kv_bytes_per_token_layer"]
  return n["weight_bytes"] + batch * kv


def prefill_flops(cfg, layers, tokens):
  d, f, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
  hq, hkv, dh = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
  linear = 2 * tokens * (d * (hq + 2 * hkv) * dh + hq * dh * d + 3 * d * f)
  types = cfg.resolved_layer_types()[:layers]
  attn = 0
  for t in types:
    w = cfg.sliding_window if t == "sliding_attention" else tokens
    pairs = sum(min(i + 1, w) for i in range(tokens))
    attn += 4 * dh * hq * pairs
  return layers * linear + attn + 2 * d * v


def reference_arm(args):
  """Runs nothing: the reference installs only without its dependencies and cannot be imported
  (`pip install --no-deps --target baseline/_ref` works; `import simply.model_lib` needs jax,
  orbax and etils, which are not installed and cannot be, and its paged attention is a TPU
  Pallas kernel)."""
  why = "baseline/_ref is absent: google-deepmind/simply was not installed"
  ref = os.path.join(ROOT, "baseline", "_ref")
  if os.path.isdir(os.path.join(ref, "simply")):
    sys.path.insert(0, ref)
    try:
      import simply.model_lib  # noqa: F401
      why = "simply imports, but its paged attention is a TPU-only Pallas kernel with no CUDA path"
    except Exception as e:  # ModuleNotFoundError: jax
      why = f"import simply.model_lib fails offline: {type(e).__name__}: {e}"
  print(json.dumps({"impl": "reference", "unavailable": why}))
  return 0


def settle(torch, seconds=0.5):
  """Filling the cache for a measurement means tens of thousands of prompt tokens at full power,
  after which the GPU runs under its power cap for some 50 ms (decode steps then take 2.5 instead
  of 2.3 ms end to end).  Half a second of rest before the warm-up steps lets the clocks settle;
  the clocks sampled during the run are in the output."""
  torch.cuda.synchronize()
  time.sleep(seconds)


BURSTS = 5  # timed bursts per decode point; the median is reported


def time_decode(engine, torch, batch, context, steps, warmup, seed, bursts=BURSTS):
  """Device time of a burst of `steps` decode steps at `batch`: the median of `bursts` bursts
  that follow one another, the last one ending at `context` cached tokens.  Returns (ms per
  step, kernel launches per step, [ms per step of every burst])."""
  import numpy as np
  from simply_b200 import StepEntry

  rng = np.random.default_rng(seed)
  vocab = engine.model.spec.vocab_size
  bursts = max(1, min(bursts, (context - warmup - 1) // steps))
  start = context - bursts * steps - warmup
  slots = [engine.open_request(f"bench{seed}_{i}") for i in range(batch)]
  chunk = 2048
  for slot in slots:
    done = 0
    while done < start:
      n = min(chunk, start - done)
      engine.step_raw([StepEntry(slot, rng.integers(0, vocab, n).tolist(), ())])
      done += n
  settle(torch)
  runner = engine._decode_runner
  params = engine.ops.pack_sample_params([0.0] * batch, [-1] * batch, [1.0] * batch, list(range(batch)),
                                         [start + 1] * batch)
  last = rng.integers(0, vocab, batch).tolist()
  toks = runner.run(slots, last, params, warmup)  # captures the graph, warms up
  params[:, 5] += warmup
  # Timed: `steps` replays back to back, `bursts` times; events bracket exactly one burst each.
  per_burst = []
  launches = 0.0
  for _ in range(bursts):
    torch.cuda.synchronize()
    launches0 = engine.ops.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    toks = runner.run(slots, toks[-1].tolist(), params, steps)
    e1.record()
    torch.cuda.synchronize()
    per_burst.append(e0.elapsed_time(e1) / steps)
    launches = (engine.ops.launches - launches0) / steps
    params[:, 5] += steps
  engine.ops.check_errors()
  for slot in slots:
    engine.close_request(slot)
  return float(np.median(per_burst)), launches, per_burst


def time_kernels(engine, torch, cfg, batch, context, peaks):
  """The dominant kernels on their own, each over all layers in a row so that every launch
  streams its own weights or its own cache from memory (5 GB of weights, 5 GB of cache: far
  more than L2): the four products of a decode step, the attention of a decode step, and the
  gate-up product with its activation for a 2,048-token prompt.  Median of 5, device-timed."""
  import numpy as np
  from simply_b200 import StepEntry

  ops, dev = engine.ops, engine.device
  blocks = list(engine.model.blocks.values())

  def timed(fn, reps=5):
    fn()
    times = []
    for _ in range(reps):
      torch.cuda.synchronize()
      e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      e0.record()
      fn()
      e1.record()
      torch.cuda.synchronize()
      times.append(e0.elapsed_time(e1))
    return float(np.median(times))

  out = {}
  d, hq, dh, f = cfg.hidden_size, cfg.num_attention_heads, cfg.head_dim, cfg.intermediate_size
  x_d = torch.randn(batch, d, device=dev).to(torch.bfloat16)
  x_o = torch.randn(batch, hq * dh, device=dev).to(torch.bfloat16)
  x_f = torch.randn(batch, f, device=dev).to(torch.bfloat16)

  def products():
    for b in blocks:
      ops.linear(x_d, b.mixer.qkv_weight)
      ops.linear(x_o, b.mixer.o_proj.weight)
      ops.gated_linear(x_d, b.feed_forward.gate_up_weight, b.feed_forward.activation)
      ops.linear(x_f, b.feed_forward.down_proj.weight)

  with ops.hold_stream():
    ms = timed(products)
  weight_bytes = sum(w.numel() * 2 for b in blocks for w in (
      b.mixer.qkv_weight, b.mixer.o_proj.weight, b.feed_forward.gate_up_weight, b.feed_forward.down_proj.weight))
  gbs = weight_bytes / (ms * 1e-3) / 1e9
  out[f"decode_products_b{batch}"] = {"ms": round(ms, 4), "gbs": round(gbs, 1), "frac": round(gbs / peaks["hbm_gbs"], 4)}

  # The same four products for serving batches of 24 and 64 rows, replayed from a CUDA graph of all
  # layers (as the decode graphs run them: launch costs off the clock).  24 rows take the engine's
  # own tcgen05 product, 64 rows the library's.
  side = torch.cuda.Stream(device=dev)
  for rows in (24, 64):
    xs = [torch.randn(rows, k, device=dev).to(torch.bfloat16) for k in (d, hq * dh, f)]

    def serving_products():
      for b in blocks:
        ops.linear(xs[0], b.mixer.qkv_weight)
        ops.linear(xs[1], b.mixer.o_proj.weight)
        ops.gated_linear(xs[0], b.feed_forward.gate_up_weight, b.feed_forward.activation)
        ops.linear(xs[2], b.feed_forward.down_proj.weight)

    with torch.cuda.stream(side), ops.hold_stream():
      serving_products()
      torch.cuda.synchronize()
      graph = torch.cuda.CUDAGraph()
      graph.capture_begin()
      serving_products()
      graph.capture_end()
      ms = timed(graph.replay)
    gbs = weight_bytes / (ms * 1e-3) / 1e9
    out[f"decode_products_b{rows}"] = {"ms": round(ms, 4), "gbs": round(gbs, 1), "frac": round(gbs / peaks["hbm_gbs"], 4)}

  # Attention of a decode step: the cache is made to hold the context without computing it
  # (the kernel's time does not depend on what the pages hold).
  slots = [engine.open_request(f"k{i}") for i in range(batch)]
  for s in slots:
    engine.cache.extend([(s, context - 1)])
  ctx = engine._prepare([StepEntry(s, [0], (0,)) for s in slots])
  q = torch.randn(batch, hq, dh, device=dev).to(torch.bfloat16)
  calls = [(engine.caches[name], engine.model.blocks[call.layer].mixer)
           for call, name in zip(engine.model.spec.run_order, engine.model.cache_names)]

  def attention():
    for cache, m in calls:
      ops.paged_attention(q, cache.storage, ctx.block_tables[cache.group], ctx, num_heads=m.num_heads,
                          num_kv_heads=m.num_kv_heads, head_dim=m.head_dim, logit_softcap=m.logit_softcap,
                          window=m.window)

  with ops.hold_stream():
    ms = timed(attention)
  kv_bytes = decode_bytes(cfg, len(blocks), batch, context) - model_numbers(cfg, len(blocks))["weight_bytes"]
  gbs = kv_bytes / (ms * 1e-3) / 1e9
  out[f"decode_attention_b{batch}"] = {"ms": round(ms, 4), "gbs": round(gbs, 1), "frac": round(gbs / peaks["hbm_gbs"], 4)}
  ops.check_errors()
  for s in slots:
    engine.close_request(s)

  tokens = 2048
  x_p = torch.randn(tokens, d, device=dev).to(torch.bfloat16)

  def gate_up():
    for b in blocks:
      ops.gated_linear(x_p, b.feed_forward.gate_up_weight, b.feed_forward.activation)

  with ops.hold_stream():
    ms = timed(gate_up)
  tflops = 2 * tokens * d * 2 * f * len(blocks) / (ms * 1e-3) / 1e12
  out[f"prefill_gate_up_{tokens}"] = {"ms": round(ms, 4), "tflops": round(tflops, 1),
                                      "frac": round(tflops / peaks["bf16_tflops"], 4)}
  return out


def time_serving(engine, torch, cfg, requests=128, prompt=512, out=128):
  """A serving-like run through `Engine.generate`, host tokens in and out: `requests` greedy
  requests with prompts of prompt/2 to 3*prompt/2 tokens and out/2 to 3*out/2 generated tokens,
  batched continuously over the engine's slots (prompt portions beside decoding requests, decode
  steps from graphs).  Run twice; the second run, whose graphs exist, is the one reported."""
  import numpy as np
  from simply_b200 import SamplingParams

  rng = np.random.default_rng(7)
  result = {}
  for _ in range(2):
    prompts = [rng.integers(0, cfg.vocab_size, int(k)).tolist() for k in rng.integers(prompt // 2, prompt * 3 // 2, requests)]
    params = [SamplingParams(temperature=0.0, max_decode_steps=int(k), stop_token_ids=())
              for k in rng.integers(out // 2, out * 3 // 2, requests)]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    results = engine.generate(prompts, params)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    tokens_in = sum(len(p) for p in prompts)
    tokens_out = sum(len(r.output_token_ids) for r in results)
    result = {"serve_requests": requests, "serve_prompt_tokens": tokens_in, "serve_output_tokens": tokens_out,
              "serve_seconds": round(seconds, 3), "serve_output_tok_s": round(tokens_out / seconds, 1),
              "serve_total_tok_s": round((tokens_in + tokens_out) / seconds, 1)}
  return result


def profile_step(engine, torch, cfg, args, context):
  """One eager step for a profiler.  The cache is made to *hold* the context without
  computing it (attention time does not depend on the cache's contents), so that few
  launches precede the profiled ones."""
  import numpy as np
  from simply_b200 import StepEntry

  rng = np.random.default_rng(3)
  if args.profile == "mixed":
    # A serving step: every other slot decodes one token at a context of a few hundred, beside
    # the 600-token prompt of a request that has just been admitted.
    slots = [engine.open_request(f"p{i}") for i in range(args.batch - 1)]
    engine.cache.extend([(s, int(n)) for s, n in zip(slots, rng.integers(300, 900, len(slots)))])
    new = engine.open_request("new")
    entries = [StepEntry(s, [int(rng.integers(0, cfg.vocab_size))], (0,)) for s in slots]
    entries.append(StepEntry(new, rng.integers(0, cfg.vocab_size, 600).tolist(), (599,)))
  elif args.profile == "decode":
    slots = [engine.open_request(f"p{i}") for i in range(args.batch)]
    engine.cache.extend([(s, context - 2) for s in slots])
    entries = [StepEntry(s, [int(rng.integers(0, cfg.vocab_size))], (0,)) for s in slots]
  else:
    slot = engine.open_request("p")
    n = min(2048, context - 1)
    entries = [StepEntry(slot, rng.integers(0, cfg.vocab_size, n).tolist(), (n - 1,))]

  def step():
    logits = engine.step_raw(entries)
    engine.ops.sample(logits, [0.0] * len(entries), [-1] * len(entries), [1.0] * len(entries),
                      [0] * len(entries), [1] * len(entries))

  if args.profile == "mixed":
    step()  # warm-up; then the same step again with the prompt under a new request
    engine.close_request(entries[-1].slot)
    new = engine.open_request("new2")
    entries = [StepEntry(e.slot, e.tokens, e.want) for e in entries[:-1]] + [StepEntry(new, entries[-1].tokens, entries[-1].want)]
  elif args.profile == "prefill":
    step()  # warm-up on the same slot is not possible for a prompt; use a second request
    engine.close_request(entries[0].slot)
    slot = engine.open_request("p2")
    entries = [StepEntry(slot, entries[0].tokens, entries[0].want)]
  else:
    step()
    entries = [StepEntry(e.slot, e.tokens, e.want) for e in entries]
  torch.cuda.synchronize()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  torch.cuda.profiler.start()
  t0 = time.perf_counter()
  e0.record()
  step()
  e1.record()
  host_ms = (time.perf_counter() - t0) * 1e3
  torch.cuda.synchronize()
  torch.cuda.profiler.stop()
  engine.ops.check_errors()
  print(f"profiled one {args.profile} step: {len(entries)} entries, context {context}, "
        f"{cfg.num_hidden_layers} layers; the host issued it in {host_ms:.2f} ms, the device took "
        f"{e0.elapsed_time(e1):.2f} ms")
  return 0


def main(argv=None):
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=32)
  ap.add_argument("--warmup", type=int, default=4)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
  ap.add_argument("--preset", default="gemma2-2b")
  ap.add_argument("--batch", type=int, default=8)
  ap.add_argument("--context", type=int, default=0, help="0: the preset's max_position_embeddings")
  ap.add_argument("--layers", type=int, default=0, help="0: all layers of the preset")
  ap.add_argument("--page-size", type=int, default=64, help="tokens per cache page")
  ap.add_argument("--skip-points", action="store_true", help="only the headline batch")
  ap.add_argument("--profile", choices=["decode", "prefill", "mixed"], default=None,
                  help="run ONE eager step of this kind between cudaProfilerStart/Stop and exit "
                       "(for ncu --profile-from-start off); prints no benchmark line")
  args = ap.parse_args(argv)
  if args.impl == "reference":
    return reference_arm(args)
  if args.gpus != 1:
    print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
    return 2
  if args.warmup < 3:
    args.warmup = 3
  if not 1 <= args.steps <= 60:
    print("bench.py: --steps must be between 1 and 60 (one burst of graph replays)")
    return 2

  import numpy as np
  import torch

  from simply_b200 import Engine, EngineConfig, SamplingParams, StepEntry, preset

  peaks, peaks_from = load_peaks()
  cfg = preset(args.preset)
  full_layers = cfg.num_hidden_layers
  layers = args.layers or full_layers
  if layers != full_layers:
    cfg = cfg.replace(num_hidden_layers=layers, layer_types=cfg.resolved_layer_types()[:layers])
  context = args.context or cfg.max_position_embeddings
  # The other decode points of each named configuration: (batch, context).  The largest model's
  # batch of 64 runs at 2,048 cached tokens (its cache at 8,192 would not fit beside the weights).
  point_table = {"gemma2-9b": ((1, context), (32, context)), "gemma2-27b": ((1, context), (64, min(context, 2048)))}
  point_list = point_table.get(args.preset, ((1, context), (64, context)))
  max_batch = 8 if args.skip_points else max(b for b, _ in point_list)
  max_batch = max(max_batch, args.batch)
  cache_tokens = max([args.batch * context] + ([] if args.skip_points else [b * c for b, c in point_list]))
  ec = EngineConfig(activation_dtype="bfloat16", page_size=args.page_size, batch_size=max_batch, max_seq_len=context,
                    max_cache_tokens=cache_tokens, max_num_issue_tokens=2048, intermediate_steps=1)
  t0 = time.time()
  engine = Engine.from_config(cfg, seed=0, engine_config=ec, matrix_std=0.02, scale_std=0.0)
  torch.cuda.synchronize()
  setup_s = time.time() - t0

  if args.profile:
    return profile_step(engine, torch, cfg, args, context)

  sampler = ClockSampler()
  sampler.start()

  # ---- decode, device-timed ----------------------------------------------------------
  ms_step, launches, bursts_ms = time_decode(engine, torch, args.batch, context, args.steps, args.warmup, seed=1)
  value = args.batch / (ms_step * 1e-3)

  # ---- end to end through the public entry point (next, while the GPU is in the same state) ---
  # The prompts are computed under the engine's own token budget, in steps that also decode for
  # the requests whose prompts are done; the requests therefore begin to decode a few steps apart
  # and are a few tokens apart in the timed steps (`slack`), all of them just below the full context.
  rng = np.random.default_rng(4)
  slack = -(-context // ec.max_num_issue_tokens) * args.batch + 8
  start = context - args.steps - args.warmup - slack
  prompts = [rng.integers(0, cfg.vocab_size, start).tolist() for _ in range(args.batch)]
  sp = SamplingParams(temperature=0.0, max_decode_steps=args.steps + args.warmup + slack, stop_token_ids=())
  requests = [engine.add_request(p, sp) for p in prompts]
  while any(not r.is_decoding for r in requests):
    engine.step()  # prompt portions beside decoded tokens (untimed)
  settle(torch)
  for _ in range(args.warmup):
    engine.step()
  torch.cuda.synchronize()
  runner = engine._decode_runner
  h2d0, d2h0 = runner.h2d_bytes, runner.d2h_bytes
  t0 = time.perf_counter()
  e2e_steps = 0
  step_ends = []
  while e2e_steps < args.steps:
    engine.step()
    e2e_steps += 1
    step_ends.append(time.perf_counter())
  torch.cuda.synchronize()
  e2e_s = time.perf_counter() - t0
  assert all(r.is_decoding for r in requests), "a request ended inside the timed steps"
  step_ms = np.diff(np.array([t0] + step_ends)) * 1e3
  h2d = (runner.h2d_bytes - h2d0) // max(e2e_steps, 1)  # counted where the copies are made
  d2h = (runner.d2h_bytes - d2h0) // max(e2e_steps, 1)
  for r in requests:
    engine.cancel(r.request_id)
  e2e_value = args.batch * e2e_steps / e2e_s

  points = {}
  kernels = {}
  if not args.skip_points:
    for b, c in point_list:
      ms_b, _, _ = time_decode(engine, torch, b, c, args.steps, args.warmup, seed=10 + b)
      name = f"decode_b{b}" if c == context else f"decode_b{b}_ctx{c}"
      points[name] = round(b / (ms_b * 1e-3), 1)
      points[f"{name}_ms"] = round(ms_b, 4)
      points[f"{name}_hbm_frac"] = round(decode_bytes(cfg, layers, b, c) / (ms_b * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
    for c in (1024, 4096):
      if c < context:
        ms_c, _, _ = time_decode(engine, torch, args.batch, c, args.steps, args.warmup, seed=20 + c)
        name = f"decode_b{args.batch}_ctx{c}"
        points[name] = round(args.batch / (ms_c * 1e-3), 1)
        points[f"{name}_ms"] = round(ms_c, 4)
        points[f"{name}_hbm_frac"] = round(decode_bytes(cfg, layers, args.batch, c) / (ms_c * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
    kernels = time_kernels(engine, torch, cfg, args.batch, context, peaks)

  # ---- prefill: one 2,048-token prompt in one step --------------------------------------
  rng = np.random.default_rng(5)
  p_tokens = min(2048, context)
  prompt = rng.integers(0, cfg.vocab_size, p_tokens).astype(np.int32)  # host tokens, as an array
  times = []
  settle(torch)
  for i in range(3 + 5):
    slot = engine.open_request(f"prefill{i}")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if i >= 3:
      settle(torch, 0.25)  # a prompt arrives on its own: each timed step starts from settled clocks
    torch.cuda.synchronize()
    e0.record()
    engine.step_raw([StepEntry(slot, prompt, (p_tokens - 1,))])
    e1.record()
    torch.cuda.synchronize()
    if i >= 3:
      times.append(e0.elapsed_time(e1))
    engine.close_request(slot)
  prefill_ms = float(np.median(times))
  flops = prefill_flops(cfg, layers, p_tokens)
  prefill = {"value": round(p_tokens / (prefill_ms * 1e-3), 1), "tokens": p_tokens, "ms": round(prefill_ms, 3),
             "frac": round(flops / (prefill_ms * 1e-3) / 1e12 / peaks["bf16_tflops"], 4)}

  if not args.skip_points:
    # Longer prompts in one step each (attention's share grows with the length).
    for tokens in (4096, 8192):
      if tokens > context:
        continue
      long_prompt = rng.integers(0, cfg.vocab_size, tokens).astype(np.int32)
      times = []
      for i in range(1 + 3):
        slot = engine.open_request(f"prefill{tokens}_{i}")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if i >= 1:
          settle(torch, 0.25)
        torch.cuda.synchronize()
        e0.record()
        engine.step_raw([StepEntry(slot, long_prompt, (tokens - 1,))])
        e1.record()
        torch.cuda.synchronize()
        if i >= 1:
          times.append(e0.elapsed_time(e1))
        engine.close_request(slot)
      ms = float(np.median(times))
      points[f"prefill_{tokens}_ms"] = round(ms, 3)
      points[f"prefill_{tokens}_frac"] = round(prefill_flops(cfg, layers, tokens) / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"], 4)
    budget = engine.scheduler.max_num_issue_tokens
    engine.scheduler.max_num_issue_tokens = 2048
    points.update(time_serving(engine, torch, cfg))
    engine.scheduler.max_num_issue_tokens = budget

  metric_name = {"gemma2-2b": "Gemma 2 2B", "gemma2-9b": "Gemma 2 9B", "gemma2-27b": "Gemma 2 27B"}.get(args.preset, args.preset)
  clocks = sampler.stop()
  step_bytes = decode_bytes(cfg, layers, args.batch, context)
  achieved = step_bytes / (ms_step * 1e-3) / 1e9
  n = model_numbers(cfg, layers)
  out = {
      "metric": f"decode tok/s @ batch {args.batch}, {context}-token context ({metric_name}, 1 B200)",
      "value": round(value, 1),
      "unit": "tokens/s",
      "n_gpus": 1,
      "steps": args.steps,
      "warmup": args.warmup,
      "ms_per_step": round(ms_step, 4),
      "higher_is_better": True,
      "scaling": "weak",
      "vs_baseline": None,
      "dtype": "bf16",
      "data": "synthetic: random bf16 weights N(0, 0.02) seed 0, uniform random token ids",
      "impl": "ours",
      "config": {
          "model": args.preset, "layers": layers, "layers_full": full_layers, "width": cfg.hidden_size,
          "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
          "ffn": cfg.intermediate_size, "vocab": cfg.vocab_size, "window": cfg.sliding_window,
          "global_batch": args.batch, "seq_len": context, "page_size": args.page_size, "parallelism": "1 GPU",
          "l2": "inputs larger than L2", "peaks": peaks_from, "params": n["params"],
          "timed": f"median of {len(bursts_ms)} bursts of {args.steps} steps",
      },
      "bursts_ms_per_step": [round(b, 4) for b in bursts_ms],
      "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
              "d2h_bytes_per_step": d2h, "steps": e2e_steps,
              "median_step_ms": round(float(np.median(step_ms)), 4), "max_step_ms": round(float(step_ms.max()), 4)},
      "gpu_launches": int(round(launches * args.steps)),
      "prefill": prefill,
      "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                   "frac": round(achieved / peaks["hbm_gbs"], 4)},
      "points": points,
      "kernels": kernels,
      "clocks": clocks,
      "setup_s": round(setup_s, 1),
  }
  print(json.dumps(out))
  return 0


if __name__ == "__main__":
  sys.exit(main())
