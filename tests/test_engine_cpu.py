"""The engine's host side on a machine without a GPU: the cache manager, the step function,
the scheduler and replay run with the plain-PyTorch kernel table (tests/reference_ops.py)
and must reproduce the plain NumPy model under every way of cutting the work."""

import numpy as np
import pytest
import torch

from simply_b200 import Engine, EngineConfig, SamplingParams, StepEntry
from simply_b200.engine.replay import engine_for_replay
from tests import replay_cases as cases
from tests import trace_util
from tests.plain import gemma2_plain as plain_lib
from tests.plain.gemma2_plain import PlainGemma2
from tests.reference_ops import ReferenceOps
from tests.tiny_models import write_tiny
from tests.tolerances import assert_logits_close


@pytest.fixture(scope="module")
def models(tmp_path_factory):
  root = tmp_path_factory.mktemp("models")
  out = {}
  for which in ("a", "b"):
    folder = write_tiny(which, root, "bfloat16")
    plain = PlainGemma2(folder)
    requests = cases.make_requests(which, plain.cfg["vocab_size"])
    out[which] = (folder, plain, requests, {rid: plain.forward(t) for rid, t in requests.items()})
  return out


def cpu_engine(folder, dtype="float32", **kw):
  kw.setdefault("page_size", 8)
  kw.setdefault("batch_size", 4)
  kw.setdefault("max_seq_len", 256)
  return Engine.from_folder(folder, EngineConfig(activation_dtype=dtype, **kw),
                            ops=ReferenceOps(getattr(torch, dtype)))


@pytest.mark.parametrize("dtype,page", [("float32", 64), ("float32", 4), ("bfloat16", 8)])
@pytest.mark.parametrize("which", ["a", "b"])
def test_replay_four_ways(models, tmp_path, which, dtype, page):
  folder, plain, requests, expected = models[which]
  steps = cases.combined_trace(requests)
  eng = engine_for_replay(folder, dtype, trace_util.tokens_needed(steps, page), page, poison_freed_pages=True,
                          ops=ReferenceOps(getattr(torch, dtype)))
  trace_util.run_in_process(eng, steps, str(tmp_path))
  eng.cache.check_invariants()
  assert eng.cache.all_pages_free()  # every request was ended
  cases.compare(trace_util.collect(steps, str(tmp_path), plain.cfg["vocab_size"]), requests, expected, dtype)


def test_step_returns_only_wanted_rows_in_order(models):
  folder, plain, requests, expected = models["a"]
  eng = cpu_engine(folder)
  (r0, t0), (r1, t1) = list(requests.items())[:2]
  a, b = eng.open_request("a"), eng.open_request("b")
  assert eng.step_raw([StepEntry(a, t0[:10], ()), StepEntry(b, t1[:4], ())]) is None
  got = eng.step_raw([StepEntry(b, t1[4:9], (4, 0)), StepEntry(a, t0[10:12], (1,))]).numpy()
  want = np.stack([expected[r1][8], expected[r1][4], expected[r0][11]])
  assert_logits_close(got, want, "float32")
  with pytest.raises(ValueError, match="outside its"):
    eng.step_raw([StepEntry(a, [1, 2], (2,))])
  with pytest.raises(ValueError, match="vocabulary"):
    eng.step_raw([StepEntry(a, [10 ** 6], ())])


@pytest.mark.parametrize("which,lengths,steps,page", [("a", (5, 11, 17), 8, 4), ("b", (1, 23, 40), 12, 8)])
def test_generation_equals_plain(models, which, lengths, steps, page):
  folder, plain, _, _ = models[which]
  rng = np.random.default_rng(1)
  prompts = [rng.integers(0, plain.cfg["vocab_size"], n).tolist() for n in lengths]
  eng = cpu_engine(folder, page_size=page, max_num_issue_tokens=7)
  got = eng.generate(prompts, SamplingParams(temperature=0.0, max_decode_steps=steps, stop_token_ids=()))
  assert [r.output_token_ids for r in got] == [plain.greedy(p, steps) for p in prompts]
  got = eng.generate(prompts, SamplingParams(temperature=0.8, seed=3, max_decode_steps=steps, stop_token_ids=()))
  assert [r.output_token_ids for r in got] == [plain.sample(p, steps, 0.8, 3) for p in prompts]
  eng.cache.check_invariants()


def test_logprobs_and_default_seeds(models):
  """simply/utils/sampling_lib.py:540-601: every output token comes with its log-probability under
  the distribution it was drawn from (0 for greedy requests).  Requests without a seed each get
  one of their own, so equal prompts draw different samples; an explicit seed repeats itself."""
  folder, plain, _, _ = models["b"]
  rng = np.random.default_rng(6)
  prompts = [rng.integers(0, plain.cfg["vocab_size"], n).tolist() for n in (12, 31)]
  eng = cpu_engine(folder, page_size=8, max_num_issue_tokens=16)
  sp = SamplingParams(temperature=0.7, top_k=30, top_p=0.9, seed=5, max_decode_steps=6, stop_token_ids=(),
                      logprobs=True)
  for p, r in zip(prompts, eng.generate(prompts, sp)):
    assert r.output_token_ids == plain.sample(p, 6, 0.7, 5, top_k=30, top_p=0.9)
    logits = plain.forward(p + r.output_token_ids)
    want = [plain_lib.token_logprob(logits[len(p) - 1 + i], t, 0.7, 30, 0.9) for i, t in enumerate(r.output_token_ids)]
    np.testing.assert_allclose(r.output_token_logprobs, want, atol=2e-4)
    assert all(v <= 0 for v in r.output_token_logprobs)
  greedy = eng.generate(prompts, SamplingParams(temperature=0.0, max_decode_steps=4, stop_token_ids=(), logprobs=True))
  assert all(r.output_token_logprobs == [0.0] * 4 for r in greedy)
  assert eng.generate(prompts[:1], SamplingParams(max_decode_steps=2))[0].output_token_logprobs is None
  # no seed: the same prompt twice draws two different continuations; with a seed, the same one
  same = [prompts[0], prompts[0]]
  a, b = eng.generate(same, SamplingParams(temperature=1.0, max_decode_steps=12, stop_token_ids=()))
  assert a.output_token_ids != b.output_token_ids
  a, b = eng.generate(same, SamplingParams(temperature=1.0, seed=9, max_decode_steps=12, stop_token_ids=()))
  assert a.output_token_ids == b.output_token_ids == plain.sample(prompts[0], 12, 1.0, 9)


def test_score_tokens(models):
  """simply/model_lib.py:4995-5036: the log-likelihood of each token given those before it, under
  the plain softmax or under sampling masks; greedy scores the argmax 0 and anything else -inf."""
  folder, plain, _, _ = models["b"]
  toks = np.random.default_rng(8).integers(0, plain.cfg["vocab_size"], 37).tolist()
  eng = cpu_engine(folder, page_size=8)
  logits = plain.forward(toks)
  want = [plain_lib.token_logprob(logits[i], toks[i + 1], 1.0, -1, 1.0) for i in range(len(toks) - 1)]
  got = eng.score_tokens(toks, rows_per_step=7)  # in portions, through the cache
  np.testing.assert_allclose(got, want, atol=2e-4)
  assert len(got) == len(toks) - 1 and eng.cache.all_pages_free()
  masked = eng.score_tokens(toks, SamplingParams(temperature=0.7, top_k=5))
  want = [plain_lib.token_logprob(logits[i], toks[i + 1], 0.7, 5, 1.0) for i in range(len(toks) - 1)]
  assert [np.isinf(a) for a in masked] == [np.isinf(b) for b in want] and any(np.isinf(want))
  np.testing.assert_allclose([a for a in masked if np.isfinite(a)], [b for b in want if np.isfinite(b)], atol=2e-4)
  greedy_path = toks[:5] + plain.greedy(toks[:5], 6)
  assert eng.score_tokens(greedy_path, SamplingParams(temperature=0.0))[4:] == [0.0] * 6
  assert eng.score_tokens([3], None) == []


def test_eos_ends_a_request(models):
  folder, plain, _, _ = models["a"]
  prompt = [3, 1, 4, 1, 5]
  first = plain.greedy(prompt, 3)
  eng = cpu_engine(folder)
  r = eng.generate([prompt], SamplingParams(temperature=0.0, max_decode_steps=9, stop_token_ids=(first[2],)))[0]
  assert r.output_token_ids == first[:first.index(first[2]) + 1] and r.finish_reason == "eos" and not r.is_truncated


def test_preemption_gives_the_same_tokens(models):
  folder, plain, _, _ = models["b"]
  rng = np.random.default_rng(9)
  prompts = [rng.integers(0, 1000, n).tolist() for n in (20, 25, 30)]
  sp = SamplingParams(temperature=0.9, seed=2, max_decode_steps=30, stop_token_ids=())
  roomy = cpu_engine(folder).generate(prompts, sp)
  tight_engine = cpu_engine(folder, max_cache_tokens=120)
  tight = tight_engine.generate(prompts, sp)
  assert [r.output_token_ids for r in tight] == [r.output_token_ids for r in roomy]
  assert sum(r.num_preemptions for r in tight) > 0
  assert tight_engine.cache.all_pages_free()


def test_the_package_has_no_cpu_path():
  if torch.cuda.is_available():
    pytest.skip("this machine has a GPU")
  from simply_b200.kernels.ops import CudaOps, KernelError
  with pytest.raises(KernelError, match="no CPU path"):
    CudaOps(torch.bfloat16)


def test_decode_graph_batch_sizes():
  """The batch sizes decode graphs are captured for: never below the live requests, few of them,
  less than as many padded rows as live ones, at most half as many from 16 on, and not beyond the engine's slots."""
  from types import SimpleNamespace
  from simply_b200.engine.decode_graph import DecodeRunner

  def bucket(live, slots):
    fake = SimpleNamespace(engine=SimpleNamespace(cache=SimpleNamespace(max_slots=slots)))
    return DecodeRunner.batch_bucket(fake, live)

  sizes = {bucket(n, 256) for n in range(1, 257)}
  assert len(sizes) <= 16
  for n in range(1, 257):
    b = bucket(n, 256)
    assert n <= b <= max(2 * n - 1, 1) and (n < 16 or b <= n * 3 // 2)
  assert bucket(37, 40) == 40 and bucket(41, 40) == 41 and bucket(5, 6) == 6
