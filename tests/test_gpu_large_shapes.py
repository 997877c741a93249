"""The layer sizes of the large configurations, two layers deep: the bfloat16 path (tcgen05 prefill
attention, TMA-fed decode attention, weight-streaming products with their fused epilogues, library
products for the long portions) against the true 32-bit path of the same engine, which the tiny
configurations tie to the plain model.  The tiny configurations cannot reach these kernels' large
tiles (head sizes 128 and 256, rows of thousands of values, prompts of thousands of tokens)."""

import numpy as np
import pytest

from simply_b200 import Engine, EngineConfig, StepEntry, preset
from tests.tolerances import assert_logits_close

pytestmark = pytest.mark.gpu


def run(cfg, dtype, tokens, other, prompt_len):
  eng = Engine.from_config(cfg, 0, EngineConfig(activation_dtype=dtype, batch_size=2, max_seq_len=8192,
                                                max_cache_tokens=8192, use_cuda_graphs=False),
                           matrix_std=0.03, scale_std=0.1)
  a, b = eng.open_request("a"), eng.open_request("b")
  rows = []
  # a long prompt in two portions (the second one attends to the first through the cache) ...
  rows.append(eng.step_raw([StepEntry(a, tokens[:2048], (0, 1000, 2047))]))
  rows.append(eng.step_raw([StepEntry(a, tokens[2048:prompt_len], (0, prompt_len - 2049))]))
  # ... then single tokens, the first few beside a second request's prompt portion and tokens
  rows.append(eng.step_raw([StepEntry(a, [tokens[prompt_len]], (0,)), StepEntry(b, other[:300], (299,))]))
  for i in range(1, 12):
    rows.append(eng.step_raw([StepEntry(a, [tokens[prompt_len + i]], (0,)), StepEntry(b, [other[299 + i]], (0,))]))
  eng.ops.check_errors()
  return np.concatenate([r.float().cpu().numpy() for r in rows])


@pytest.mark.parametrize("name", ["gemma2-2b", "gemma2-27b"])
def test_bfloat16_follows_float32_at_large_layer_sizes(name):
  cfg = preset(name).replace(num_hidden_layers=2, vocab_size=20000)
  rng = np.random.default_rng(3)
  prompt_len = 2048 + 901  # beyond one portion, not a multiple of a tile
  tokens = rng.integers(0, cfg.vocab_size, prompt_len + 16).tolist()
  other = rng.integers(0, cfg.vocab_size, 320).tolist()
  got = run(cfg, "bfloat16", tokens, other, prompt_len)
  want = run(cfg, "float32", tokens, other, prompt_len)
  assert_logits_close(got, want, "bfloat16", name)
  assert (got.argmax(-1) == want.argmax(-1)).mean() > 0.9


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
    assert eng.cache.min_free_pages() == eng.cache.num_pages
    assert all(r.finish_reason == "max_decode_steps" for r in results)
    outputs.append([r.output_token_ids for r in results])
    preemptions += sum(r.num_preemptions for r in results)
  assert outputs[1] == outputs[0] and outputs[2] == outputs[0]
  assert preemptions > 0
