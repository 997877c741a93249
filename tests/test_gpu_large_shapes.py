"""The layer sizes of the large configurations, two layers deep, against the plain model: the
bfloat16 path (tcgen05 prefill attention, TMA-fed decode attention, weight-streaming products with
their fused epilogues, library products for the long portions, decode steps replayed from CUDA
graphs) and the true 32-bit path, each compared with the plain NumPy model on the same weights.  The tiny configurations cannot reach these kernels' large tiles (head sizes
128 and 256, rows of thousands of values, prompts of thousands of tokens)."""

import gc

import numpy as np
import pytest

from simply_b200 import Engine, EngineConfig, StepEntry, preset
from simply_b200.weights import write_model_folder
from tests.plain.gemma2_plain import PlainGemma2
from tests.tolerances import assert_logits_close

pytestmark = pytest.mark.gpu

# name -> tokens of the long prompt (beyond one portion, not a multiple of a tile) and its first portion
SHAPES = {"gemma2-2b": (2048 + 453, 2048), "gemma2-9b": (2048 + 453, 2048), "gemma2-27b": (1024 + 389, 1024)}
VOCAB = 8000
SINGLE = 12  # tokens fed one by one after the prompt


def wanted(prompt_len, portion):
  """Positions of the long request whose logits are compared."""
  return [0, portion // 2, portion - 1, portion, prompt_len - 1] + list(range(prompt_len, prompt_len + SINGLE))


@pytest.fixture(scope="module", params=list(SHAPES))
def case(request, tmp_path_factory):
  """A model folder with two layers of the named configuration's sizes (one with a window, one
  without), two requests, and the plain model's logits for them."""
  name = request.param
  prompt_len, portion = SHAPES[name]
  cfg = preset(name).replace(num_hidden_layers=2, vocab_size=VOCAB)
  folder = write_model_folder(cfg, 0, str(tmp_path_factory.mktemp(name)), matrix_std=0.03, scale_std=0.1,
                              device="cuda")
  rng = np.random.default_rng(3)
  tokens = rng.integers(0, VOCAB, prompt_len + SINGLE).tolist()
  other = rng.integers(0, VOCAB, 300 + SINGLE - 1).tolist()
  plain = PlainGemma2(folder)
  want = np.concatenate([plain.forward(tokens)[wanted(prompt_len, portion)], plain.forward(other)[299:]])
  del plain
  gc.collect()
  return name, folder, tokens, other, want


def run(folder, dtype, tokens, other, prompt_len, portion, graphs):
  eng = Engine.from_folder(folder, EngineConfig(activation_dtype=dtype, batch_size=2, max_seq_len=8192,
                                                max_cache_tokens=8192, use_cuda_graphs=graphs))
  if graphs:
    eng._decode_runner.keep_logits = True
  a, b = eng.open_request("a"), eng.open_request("b")
  mine, others = [], []
  # a long prompt in two portions (the second one attends to the first through the cache) ...
  mine.append(eng.step_raw([StepEntry(a, tokens[:portion], (0, portion // 2, portion - 1))]))
  mine.append(eng.step_raw([StepEntry(a, tokens[portion:prompt_len], (0, prompt_len - portion - 1))]))
  # ... then single tokens, the first beside a second request's prompt, the others beside its single
  # tokens (steps that decode only, which run from the decode graphs when the engine has them)
  both = eng.step_raw([StepEntry(a, [tokens[prompt_len]], (0,)), StepEntry(b, other[:300], (299,))])
  mine.append(both[:1]), others.append(both[1:])
  for i in range(1, SINGLE):
    both = eng.step_raw([StepEntry(a, [tokens[prompt_len + i]], (0,)), StepEntry(b, [other[299 + i]], (0,))],
                        from_graph=graphs)
    mine.append(both[:1]), others.append(both[1:])
  eng.ops.check_errors()
  return np.concatenate([r.float().cpu().numpy() for r in mine + others])


@pytest.mark.parametrize("dtype,graphs", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
def test_large_layer_sizes_follow_the_plain_model(case, dtype, graphs):
  name, folder, tokens, other, want = case
  prompt_len, portion = SHAPES[name]
  got = run(folder, dtype, tokens, other, prompt_len, portion, graphs)
  assert_logits_close(got, want, dtype, f"{name} {dtype}")
  assert (got.argmax(-1) == want.argmax(-1)).mean() > (0.999 if dtype == "float32" else 0.9)


def test_generation_does_not_depend_on_batching_at_large_layer_sizes():
  """Forty requests through `generate` with three engines that batch them quite differently
  (slots, token budget, page size, bursts from CUDA graphs, a pool so small that requests are
  preempted): in the 32-bit path every request's tokens are the same, sampled ones included."""
  from simply_b200 import SamplingParams

  cfg = preset("gemma2-2b").replace(num_hidden_layers=2, vocab_size=8000, sliding_window=512)
  rng = np.random.default_rng(1)
  n = 40
  prompts = [rng.integers(0, cfg.vocab_size, int(k)).tolist() for k in rng.integers(1, 1200, n)]
  params = [SamplingParams(temperature=float(rng.choice([0.0, 0.8])), top_k=int(rng.choice([-1, 50])), seed=i,
                           max_decode_steps=int(rng.integers(1, 60)), stop_token_ids=()) for i in range(n)]
  engines = (
      dict(batch_size=32, use_cuda_graphs=True, intermediate_steps=4, max_num_issue_tokens=2048, max_cache_tokens=30000),
      dict(batch_size=5, use_cuda_graphs=False, intermediate_steps=1, max_num_issue_tokens=333, max_cache_tokens=8000),
      dict(batch_size=12, use_cuda_graphs=True, intermediate_steps=16, max_num_issue_tokens=900, max_cache_tokens=5000,
           page_size=16))
  outputs, preemptions = [], 0
  for kw in engines:
    eng = Engine.from_config(cfg, 0, EngineConfig(activation_dtype="float32", max_seq_len=2048, **kw),
                             matrix_std=0.04, scale_std=0.1)
    results = eng.generate(prompts, params)
    eng.ops.check_errors()
    eng.cache.check_invariants()
    assert eng.cache.all_pages_free()
    assert all(r.finish_reason == "max_decode_steps" for r in results)
    outputs.append([r.output_token_ids for r in results])
    preemptions += sum(r.num_preemptions for r in results)
  assert outputs[1] == outputs[0] and outputs[2] == outputs[0]
  assert preemptions > 0
