"""Decoding from CUDA graphs with the kernels the large configurations take, against the plain model.

The graph path is its own schedule: static work lists for the split-key attention kernel (with
filler items, and chunks that are empty at some steps of a burst), decode attention fed by TMA
(head sizes that are multiples of 64), several steps per host round trip, bursts that go on from
what the last one left on the device, graphs of several batch sizes as requests end.  Here the
logits of every replayed step are kept on the device (the decode runner's `keep_logits`) and
compared with the plain model's at the same position, teacher-forced on the tokens the engine
chose; the tokens themselves must be ones the plain model scores within the bound of the best.

Follows simply/utils/ragged_paged_attention_test.py:838-985 (continue_decode equals a dense
recomputation).
"""

import numpy as np
import pytest
import torch

from simply_b200 import Engine, EngineConfig, SamplingParams
from tests import trace_util
from tests.plain.gemma2_plain import PlainGemma2
from tests.tiny_models import write_tiny
from tests.tolerances import BF16_MAX, assert_logits_close

pytestmark = pytest.mark.gpu

# name -> (tiny configuration, changes).  Head sizes 64, 128 and 256 with groups 4, 2 and 1; windows
# shorter than a chunk of keys and longer than one.
MODELS = {
    "hd64_g4": ("a", dict(head_dim=64)),
    "hd128_g2": ("b", dict(head_dim=128, num_attention_heads=4, num_key_value_heads=2, sliding_window=150)),
    "hd256_g1": ("a", dict(head_dim=256, num_attention_heads=2, num_key_value_heads=2, sliding_window=70,
                           query_pre_attn_scalar=256)),
    "hd256_g2": ("b", dict(head_dim=256, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=3)),
}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
  root = tmp_path_factory.mktemp("graph_models")
  return {name: write_tiny(which, root / name, "bfloat16", max_position_embeddings=1024, **changes)
          for name, (which, changes) in MODELS.items()}


def record_bursts(engine):
  """Wraps the engine's burst so that every replayed step's logits are kept with the request and
  the position they belong to: {request_id: {position: row}}."""
  runner = engine._decode_runner
  assert runner is not None, "this model should decode from CUDA graphs"
  runner.keep_logits = True
  rows, bursts = {}, []
  inner = engine._decode_burst

  def burst(plan):
    before = [(e.request, len(e.request.tokens) - 1) for e in plan.entries]
    steps_before = engine.num_steps
    finished = inner(plan)
    logits = runner.last_logits.float().cpu().numpy()  # [steps, live, vocab]
    bursts.append((engine.num_steps - steps_before, len(before)))
    for j, (r, pos0) in enumerate(before):
      for i in range(logits.shape[0]):
        if pos0 + i < len(r.tokens) - 1:  # steps after the request's end computed rows nobody uses
          rows.setdefault(r.request_id, {})[pos0 + i] = logits[i, j]
    return finished

  engine._decode_burst = burst
  return rows, bursts


def check_against_plain(plain, prompts, results, rows, dtype):
  for i, (p, r) in enumerate(zip(prompts, results)):
    full = p + r.output_token_ids
    want = plain.forward(full[:-1])
    scale = np.abs(want).max()
    got = rows.get(r.request_id, {})
    # Every position after the prompt's last is a decode step; all but the few that shared a step
    # with a later request's prompt ran from a graph.
    decode_positions = set(range(len(p), len(full) - 1))
    assert set(got) <= decode_positions and len(got) >= len(decode_positions) - 3, (i, len(got), len(decode_positions))
    if got:
      positions = sorted(got)
      assert_logits_close(np.stack([got[q] for q in positions]), want[positions], dtype, f"request {i}")
    for j, tok in enumerate(r.output_token_ids):
      row = want[len(p) - 1 + j]
      assert row.max() - row[tok] <= 2 * BF16_MAX * scale, (i, j, tok, int(row.argmax()))


@pytest.mark.parametrize("burst", [1, 7, 16])
@pytest.mark.parametrize("name", list(MODELS))
def test_graph_decode_logits_follow_the_plain_model(folders, name, burst):
  """Requests of unequal length that end at different steps (so the batch shrinks through the
  graphs' sizes and bursts are resumed), contexts that cross the window, pages and key chunks."""
  plain = PlainGemma2(folders[name])
  rng = np.random.default_rng(100 * list(MODELS).index(name) + burst)
  lengths = (120, 3, 250, 61, 190)
  steps = (45, 70, 21, 33, 9)
  prompts = [rng.integers(0, plain.cfg["vocab_size"], n).tolist() for n in lengths]
  params = [SamplingParams(temperature=0.0, max_decode_steps=n, stop_token_ids=()) for n in steps]
  eng = Engine.from_folder(folders[name], EngineConfig(
      activation_dtype="bfloat16", page_size=16, batch_size=4, max_seq_len=512, intermediate_steps=burst,
      use_cuda_graphs=True))
  rows, bursts = record_bursts(eng)
  results = eng.generate(prompts, params)
  eng.ops.check_errors()
  eng.cache.check_invariants()
  assert eng.cache.all_pages_free()
  assert len({live for _, live in bursts}) >= 3  # graphs of several batch sizes were used
  if burst > 1:
    assert max(n for n, _ in bursts) > 1
  check_against_plain(plain, prompts, results, rows, "bfloat16")


def test_graph_decode_float32_logits(folders):
  """The same schedule in the 32-bit path (general attention kernel, static metadata only)."""
  plain = PlainGemma2(folders["hd64_g4"])
  rng = np.random.default_rng(5)
  prompts = [rng.integers(0, plain.cfg["vocab_size"], n).tolist() for n in (40, 130, 7)]
  params = [SamplingParams(temperature=0.0, max_decode_steps=n, stop_token_ids=()) for n in (30, 12, 50)]
  eng = Engine.from_folder(folders["hd64_g4"], EngineConfig(
      activation_dtype="float32", page_size=8, batch_size=4, max_seq_len=512, intermediate_steps=5))
  rows, _ = record_bursts(eng)
  results = eng.generate(prompts, params)
  eng.ops.check_errors()
  assert [r.output_token_ids for r in results] == [plain.greedy(p, n) for p, n in zip(prompts, (30, 12, 50))]
  check_against_plain(plain, prompts, results, rows, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_request_that_ends_inside_a_burst(folders, dtype):
  """A stop token that one request samples at the second or third step of a burst of eight: its
  slot and pages go back at once, the tokens the graph sampled for it afterwards are dropped, the
  others go on from a smaller batch; the output is that of single eager steps."""
  folder = folders["hd64_g4"]
  rng = np.random.default_rng(12)
  vocab = PlainGemma2(folder).cfg["vocab_size"]
  prompts = [rng.integers(0, vocab, n).tolist() for n in (33, 90, 14, 57)]

  def run(stops, **kw):
    eng = Engine.from_folder(folder, EngineConfig(activation_dtype=dtype, page_size=8, batch_size=4,
                                                  max_seq_len=512, **kw))
    params = [SamplingParams(temperature=0.9, seed=40 + i, max_decode_steps=30, stop_token_ids=s)
              for i, s in enumerate(stops)]
    results = eng.generate(prompts, params)
    eng.ops.check_errors()
    eng.cache.check_invariants()
    assert eng.cache.all_pages_free() and eng.cache.num_free_slots == 4
    return results

  free = run([()] * 4, use_cuda_graphs=False, intermediate_steps=1)

  def stop_inside_a_burst(output, first, last):
    # The first token comes from the prompt's step; bursts of eight then cover outputs 1..8, 9..16, ...
    # Wanted: a token whose first appearance is at the second to fourth step of a burst.
    for i in range(first, last):
      if output.index(output[i]) == i and (i - 1) % 8 in (1, 2, 3):
        return i, output[i]
    raise AssertionError("no token of this output can serve as a stop inside a burst")

  i1, stop1 = stop_inside_a_burst(free[1].output_token_ids, 9, 17)  # in the second burst
  i2, stop2 = stop_inside_a_burst(free[2].output_token_ids, 1, 9)  # in the first burst
  stops = [(), (stop1,), (stop2,), ()]
  eager = run(stops, use_cuda_graphs=False, intermediate_steps=1)
  graphs = run(stops, use_cuda_graphs=True, intermediate_steps=8)
  assert [r.output_token_ids for r in graphs] == [r.output_token_ids for r in eager]
  assert [r.finish_reason for r in graphs] == [r.finish_reason for r in eager]
  assert eager[1].finish_reason == "eos" and len(eager[1].output_token_ids) == i1 + 1
  assert eager[2].finish_reason == "eos" and len(eager[2].output_token_ids) == i2 + 1
  assert eager[0].finish_reason == eager[3].finish_reason == "max_decode_steps"


@pytest.mark.parametrize("name", ["hd64_g4", "hd128_g2", "hd256_g1"])
def test_trace_run_decodes_from_graphs(folders, tmp_path, name):
  """bin/trace_run --cuda-graphs: steps that bring one token per request are replays of the decode
  graphs; the logits at every position are still the plain model's."""
  plain = PlainGemma2(folders[name])
  rng = np.random.default_rng(21)
  requests = {f"r{i}": rng.integers(0, plain.cfg["vocab_size"], n).tolist() for i, n in enumerate((140, 75, 200))}
  steps = []
  for mode, build in (("tail", trace_util.prefill_then_decode), ("mixed", trace_util.mixed)):
    for s in build({f"{mode}:{rid}": toks for rid, toks in requests.items()}):
      steps.append(dict(s, step=len(steps)))
  single = [s for s in steps if all(len(e["tokens"]) == 1 for e in s["entries"])]
  assert len(single) > 60 and any(len(s["entries"]) > 1 for s in single)
  out_dir = str(tmp_path / "out")
  trace_util.run_tool(folders[name], "bfloat16", steps, out_dir, trace_util.tokens_needed(steps, 64),
                      extra=("--cuda-graphs",))
  got = trace_util.collect(steps, out_dir, plain.cfg["vocab_size"])
  for key, rows in sorted(got.items()):
    toks = requests[key.split(":")[1]]
    assert sorted(rows) == list(range(len(toks)))
    assert_logits_close(np.stack([rows[p] for p in sorted(rows)]), plain.forward(toks), "bfloat16", key)
