"""bin/trace_run on the GPU, as a user runs it, against the plain model: every request
whole; most of it in one step and the last 32 tokens one by one; in portions of changing
size; and mixed with other requests in a pool so small that pages are used again."""

import os

import numpy as np
import pytest

from tests import replay_cases as cases
from tests import trace_util
from tests.plain.gemma2_plain import PlainGemma2
from tests.tiny_models import write_tiny

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
  root = tmp_path_factory.mktemp("models")
  out = {}
  for which in ("a", "b"):
    folder = write_tiny(which, root, "bfloat16")
    plain = PlainGemma2(folder)
    requests = cases.make_requests(which, plain.cfg["vocab_size"])
    expected = {rid: plain.forward(toks) for rid, toks in requests.items()}
    out[which] = (folder, plain.cfg["vocab_size"], requests, expected)
  # The same two with head sizes of 64 and 128 and groups that divide 128: these sizes take the
  # kernels that the large configurations take (tcgen05 prefill attention, decode attention fed by
  # TMA), which head sizes of 16 and 32 do not.
  wide = {"a": dict(head_dim=64), "b": dict(head_dim=128, num_attention_heads=4, num_key_value_heads=2)}
  for which, changes in wide.items():
    folder = write_tiny(which, root / "wide", "bfloat16", **changes)
    plain = PlainGemma2(folder)
    requests = cases.make_requests(which, plain.cfg["vocab_size"])
    expected = {rid: plain.forward(toks) for rid, toks in requests.items()}
    out[which + "_wide"] = (folder, plain.cfg["vocab_size"], requests, expected)
  return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b"])
def test_trace_run_four_ways(models, tmp_path, which, dtype):
  folder, vocab, requests, expected = models[which]
  steps = cases.combined_trace(requests)
  out_dir = str(tmp_path / "out")
  trace_util.run_tool(folder, dtype, steps, out_dir, trace_util.tokens_needed(steps, 64))
  cases.compare(trace_util.collect(steps, out_dir, vocab), requests, expected, dtype)


@pytest.mark.parametrize("which", ["a_wide", "b_wide"])
def test_trace_run_four_ways_with_the_large_models_kernels(models, tmp_path, which):
  folder, vocab, requests, expected = models[which]
  steps = cases.combined_trace(requests)
  out_dir = str(tmp_path / "out")
  trace_util.run_tool(folder, "bfloat16", steps, out_dir, trace_util.tokens_needed(steps, 64))
  cases.compare(trace_util.collect(steps, out_dir, vocab), requests, expected, "bfloat16")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_small_pages_poisoned(models, tmp_path, dtype):
  """Pages of 8 tokens, freed pages filled with NaN, the pool exactly as large as the
  trace needs: a read of a page that was given back, or a stale block-table entry, shows."""
  folder, vocab, requests, expected = models["b"]
  steps = cases.combined_trace(requests, modes=("mixed", "portions"))
  out_dir = str(tmp_path / "out")
  trace_util.run_tool(folder, dtype, steps, out_dir, trace_util.tokens_needed(steps, 8),
                      extra=("--page-size", "8", "--poison-freed-pages"))
  cases.compare(trace_util.collect(steps, out_dir, vocab), requests, expected, dtype)
