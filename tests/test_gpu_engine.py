"""Generation through the public entry point on the GPU, against the plain model."""

import numpy as np
import pytest
import torch

from simply_b200 import Engine, EngineConfig, SamplingParams, StepEntry
from tests.plain.gemma2_plain import PlainGemma2
from tests.tiny_models import write_tiny
from tests.tolerances import assert_logits_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
  root = tmp_path_factory.mktemp("models")
  return {w: write_tiny(w, root, "bfloat16") for w in ("a", "b")}


def engine_for(folder, dtype, **kw):
  kw.setdefault("page_size", 8)
  kw.setdefault("batch_size", 4)
  kw.setdefault("max_seq_len", 256)
  return Engine.from_folder(folder, EngineConfig(activation_dtype=dtype, **kw))


def prompts_for(plain, lengths, seed=1):
  rng = np.random.default_rng(seed)
  return [rng.integers(0, plain.cfg["vocab_size"], n).tolist() for n in lengths]


@pytest.mark.parametrize("which,lengths,steps", [("a", (5, 11, 17), 8), ("b", (1, 23, 40), 12)])
def test_greedy_generation_float32_equals_plain(folders, which, lengths, steps):
  plain = PlainGemma2(folders[which])
  prompts = prompts_for(plain, lengths)
  want = [plain.greedy(p, steps) for p in prompts]
  for graphs in (True, False):
    eng = engine_for(folders[which], "float32", use_cuda_graphs=graphs)
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_decode_steps=steps, stop_token_ids=()))
    eng.ops.check_errors()
    assert [r.output_token_ids for r in got] == want
    assert all(r.finish_reason == "max_decode_steps" for r in got)
    eng.cache.check_invariants()


def test_temperature_sampling_float32_equals_plain(folders):
  plain = PlainGemma2(folders["b"])
  prompts = prompts_for(plain, (1, 23, 40))
  want = [plain.sample(p, 12, 0.8, 3) for p in prompts]
  # prompts cut into portions of 7 and mixed with decoding requests in one batch
  eng = engine_for(folders["b"], "float32", max_num_issue_tokens=7)
  got = eng.generate(prompts, SamplingParams(temperature=0.8, seed=3, max_decode_steps=12, stop_token_ids=()))
  assert [r.output_token_ids for r in got] == want
  # top-k and top-p as well
  want = [plain.sample(p, 6, 1.3, 11, top_k=20, top_p=0.9) for p in prompts]
  got = eng.generate(prompts, SamplingParams(temperature=1.3, seed=11, top_k=20, top_p=0.9, max_decode_steps=6,
                                             stop_token_ids=()))
  assert [r.output_token_ids for r in got] == want


@pytest.mark.parametrize("which", ["a", "b"])
def test_bfloat16_generation_follows_the_plain_model(folders, which):
  """bfloat16 may turn a near-tie, so compare teacher-forced: the engine's greedy choice at
  every step must be a token whose plain logit is within the bfloat16 bound of the best."""
  plain = PlainGemma2(folders[which])
  prompts = prompts_for(plain, (9, 30, 70))
  eng = engine_for(folders[which], "bfloat16")
  got = eng.generate(prompts, SamplingParams(temperature=0.0, max_decode_steps=24, stop_token_ids=()))
  eng.ops.check_errors()
  for p, r in zip(prompts, got):
    full = p + r.output_token_ids
    logits = plain.forward(full[:-1])
    scale = np.abs(logits).max()
    for i, tok in enumerate(r.output_token_ids):
      row = logits[len(p) - 1 + i]
      assert row.max() - row[tok] <= 2 * 3e-2 * scale, (i, tok, int(row.argmax()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_replay_and_bursts_equal_plain_steps(folders, dtype):
  plain = PlainGemma2(folders["b"])
  prompts = prompts_for(plain, (3, 18, 33, 50), seed=4)
  sp = SamplingParams(temperature=0.7, seed=5, max_decode_steps=40, stop_token_ids=())
  outs = []
  for graphs, burst in ((False, 1), (True, 1), (True, 7)):
    eng = engine_for(folders["b"], dtype, use_cuda_graphs=graphs, intermediate_steps=burst)
    outs.append([r.output_token_ids for r in eng.generate(prompts, sp)])
    eng.ops.check_errors()
    eng.cache.check_invariants()
  assert outs[0] == outs[1] == outs[2]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_logits(folders, dtype):
  """One request decoded token by token far beyond the window and over many pages, logits
  compared at every step."""
  plain = PlainGemma2(folders["a"])
  toks = prompts_for(plain, (200,), seed=8)[0]
  want = plain.forward(toks)
  eng = engine_for(folders["a"], dtype, page_size=4, max_cache_tokens=256)
  slot = eng.open_request()
  rows = [eng.step_raw([StepEntry(slot, toks[:3], (0, 1, 2))])]
  rows += [eng.step_raw([StepEntry(slot, [t], (0,))]) for t in toks[3:]]
  eng.ops.check_errors()
  assert_logits_close(torch.cat(rows).cpu().numpy(), want, dtype, "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(folders, dtype):
  plain = PlainGemma2(folders["b"])
  for n in (1, 2, 3):
    toks = prompts_for(plain, (n,), seed=20 + n)[0]
    eng = engine_for(folders["b"], dtype)
    slot = eng.open_request()
    got = eng.step_raw([StepEntry(slot, toks, tuple(range(n)))]).cpu().numpy()
    assert_logits_close(got, plain.forward(toks), dtype, f"{n} tokens")


def test_preemption_gives_the_same_tokens(folders):
  """So few pages that decoding requests must take pages from the youngest; the output is
  what an engine with room produces."""
  plain = PlainGemma2(folders["b"])
  prompts = prompts_for(plain, (20, 25, 30), seed=9)
  sp = SamplingParams(temperature=0.9, seed=2, max_decode_steps=30, stop_token_ids=())
  roomy = engine_for(folders["b"], "float32").generate(prompts, sp)
  tight_engine = engine_for(folders["b"], "float32", max_cache_tokens=120)
  tight = tight_engine.generate(prompts, sp)
  assert [r.output_token_ids for r in tight] == [r.output_token_ids for r in roomy]
  assert sum(r.num_preemptions for r in tight) > 0
  tight_engine.cache.check_invariants()
  assert tight_engine.cache.all_pages_free()


@pytest.mark.parametrize("seed", list(range(8)))
def test_random_workloads_float32_equal_plain(folders, seed):
  """Random mixes of what the host side of decoding can meet: page sizes, bursts of several steps,
  small token budgets, pools so small that requests are preempted, requests of unequal length that
  finish at different steps (so that graphs of several batch sizes are used and resumed).  Every
  token must be the plain model's."""
  rng = np.random.default_rng(100 + seed)
  which = "ab"[seed % 2]
  plain = PlainGemma2(folders[which])
  lengths = [int(n) for n in rng.integers(1, 60, size=int(rng.integers(3, 7)))]
  steps = [int(n) for n in rng.integers(1, 40, size=len(lengths))]
  prompts = prompts_for(plain, lengths, seed=50 + seed)
  sampled = seed >= 2
  params = [SamplingParams(temperature=0.7 if sampled else 0.0, seed=seed * 10 + i, max_decode_steps=n, stop_token_ids=())
            for i, n in enumerate(steps)]
  want = [plain.sample(p, n, 0.7, seed * 10 + i) if sampled else plain.greedy(p, n)
          for i, (p, n) in enumerate(zip(prompts, steps))]
  page = int(rng.choice([4, 8, 16]))
  longest = max(l + n for l, n in zip(lengths, steps))
  eng = engine_for(folders[which], "float32", page_size=page, batch_size=int(rng.integers(2, 5)),
                   intermediate_steps=int(rng.choice([1, 3, 8])), max_num_issue_tokens=int(rng.choice([5, 16, 64])),
                   max_cache_tokens=int(-(-longest // page) * page * rng.choice([1.5, 2.5, 4.0])) + 2 * page)
  got = eng.generate(prompts, params)
  eng.ops.check_errors()
  assert [r.output_token_ids for r in got] == want
  eng.cache.check_invariants()
  assert eng.cache.all_pages_free()


def test_logprobs_from_eager_steps_and_from_graph_bursts(folders):
  """Every output token's log-probability under the distribution it was drawn from, from prompt
  steps (eager) and decode bursts (CUDA graphs) alike, against the plain statement."""
  from tests.plain import gemma2_plain as plain_lib
  plain = PlainGemma2(folders["b"])
  prompts = prompts_for(plain, (7, 26, 51), seed=31)
  sp = [SamplingParams(temperature=0.8, top_k=k, top_p=p, seed=60 + i, max_decode_steps=14, stop_token_ids=(),
                       logprobs=i != 1)
        for i, (k, p) in enumerate(((-1, 1.0), (25, 1.0), (40, 0.85)))]
  eng = engine_for(folders["b"], "float32", intermediate_steps=4)
  results = eng.generate(prompts, sp)
  eng.ops.check_errors()
  assert results[1].output_token_logprobs is None
  for i in (0, 2):
    p, r = prompts[i], results[i]
    assert r.output_token_ids == plain.sample(p, 14, 0.8, 60 + i, top_k=sp[i].top_k, top_p=sp[i].top_p)
    logits = plain.forward(p + r.output_token_ids)
    want = [plain_lib.token_logprob(logits[len(p) - 1 + j], t, 0.8, sp[i].top_k, sp[i].top_p)
            for j, t in enumerate(r.output_token_ids)]
    np.testing.assert_allclose(r.output_token_logprobs, want, atol=3e-4)


def test_score_tokens_on_the_gpu(folders):
  from tests.plain import gemma2_plain as plain_lib
  plain = PlainGemma2(folders["b"])
  toks = prompts_for(plain, (90,), seed=33)[0]
  logits = plain.forward(toks)
  eng = engine_for(folders["b"], "float32")
  want = [plain_lib.token_logprob(logits[i], toks[i + 1], 1.0, -1, 1.0) for i in range(len(toks) - 1)]
  np.testing.assert_allclose(eng.score_tokens(toks, rows_per_step=32), want, atol=3e-4)
  masked = eng.score_tokens(toks, SamplingParams(temperature=0.8, top_k=10, top_p=0.9))
  want = [plain_lib.token_logprob(logits[i], toks[i + 1], 0.8, 10, 0.9) for i in range(len(toks) - 1)]
  assert [np.isinf(a) for a in masked] == [np.isinf(b) for b in want]
  np.testing.assert_allclose([a for a in masked if np.isfinite(a)], [b for b in want if np.isfinite(b)], atol=3e-4)
  greedy_path = toks[:9] + plain.greedy(toks[:9], 5)
  assert eng.score_tokens(greedy_path, SamplingParams(temperature=0.0))[8:] == [0.0] * 5
  eng.ops.check_errors()
  assert eng.cache.all_pages_free()


def test_a_float32_folder_served_in_bfloat16(tmp_path):
  """Matrices stored in 32 bits are narrowed to the activation dtype on load
  (simply/utils/checkpoint_lib.py:658-670): the engine holds bfloat16 matrices, runs the bfloat16
  kernels and gives the logits of the bfloat16 folder."""
  wide = write_tiny("b", tmp_path / "wide", "float32")
  narrow = write_tiny("b", tmp_path / "narrow", "bfloat16")
  plain = PlainGemma2(narrow)
  toks = prompts_for(plain, (45,), seed=17)[0]
  rows = {}
  for name, folder in (("wide", wide), ("narrow", narrow)):
    eng = engine_for(folder, "bfloat16")
    assert eng.model.blocks["model.layers.0"].mixer.qkv_weight.dtype == torch.bfloat16
    assert eng.model.embedding.table.dtype == torch.bfloat16
    slot = eng.open_request()
    rows[name] = eng.step_raw([StepEntry(slot, toks, tuple(range(len(toks))))]).cpu().numpy()
  assert_logits_close(rows["wide"], plain.forward(toks), "bfloat16", "float32 folder")
  # (not bit-equal: the norm scales of the float32 folder stay in 32 bits, the other folder's are rounded)
  assert_logits_close(rows["wide"], rows["narrow"], "bfloat16", "float32 folder against bfloat16 folder")
  kept = engine_for(wide, "bfloat16", keep_float32_weights=True)
  assert kept.model.blocks["model.layers.0"].mixer.qkv_weight.dtype == torch.float32


def test_engine_refuses_without_cuda_kernels(monkeypatch):
  from simply_b200.kernels import ops as ops_mod
  monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
  with pytest.raises(ops_mod.KernelError, match="no CPU path"):
    ops_mod.CudaOps(torch.bfloat16)
