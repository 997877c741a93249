"""Generality of the parts, third file: a toy model, defined here and nowhere in the package, with

  * an embedding of its own kind (token row plus a learned row per position), registered in
    EMBEDDINGS, and an output layer of its own kind (a matrix of its own, not the embedding
    table), registered in HEADS;
  * a feed-forward with routing that keeps to device tensors (every expert runs on every token,
    weighted by the router's softmax), and therefore says `graph_safe = True`;
  * two attention layers with the same window and the same group but different head sizes and
    numbers of kv heads (work lists cut for one must not serve the other);

built from a hand-written ModelSpec without a change to the package.  Because every part says it
is graph-safe, decode steps are replayed from CUDA graphs although the parts are foreign; the
logits of those replays are compared with a composition of the plain NumPy functions.  A test
fixture, not a model of anyone's."""

import numpy as np
import pytest
import torch

from simply_b200 import Engine, EngineConfig, SamplingParams, StepEntry
from simply_b200.config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from simply_b200.parts.base import Embedding, FeedForward, Head
from simply_b200.parts.model import DecoderModel
from simply_b200.registry import EMBEDDINGS, FEED_FORWARDS, HEADS
from simply_b200.weights import TensorSpec, random_tensors
from tests.plain import gemma2_plain as plain
from tests.reference_ops import ReferenceOps
from tests.tolerances import BF16_MAX, assert_logits_close

WIDTH, VOCAB, MAX_POS, HIDDEN, EXPERTS = 64, 190, 160, 32, 3
EPS, THETA, CAP = 1e-6, 5000.0, 40.0
# (query heads, kv heads, head size): the same group of 2, no window, for both layers
LAYERS = {"A": (4, 2, 32), "B": (2, 1, 64)}


class PositionedEmbedding(Embedding):
  """Token row plus a learned row for the token's position."""

  graph_safe = True

  def __init__(self, prefix, vocab_size, width, max_positions):
    self.prefix, self.vocab_size, self.width, self.max_positions = prefix, vocab_size, width, max_positions

  def tensor_specs(self):
    return [TensorSpec(f"{self.prefix}.tokens", (self.vocab_size, self.width), "matrix"),
            TensorSpec(f"{self.prefix}.positions", (self.max_positions, self.width), "matrix")]

  def bind(self, tensors, ops):
    self.tokens = tensors[f"{self.prefix}.tokens"]
    self.positions = tensors[f"{self.prefix}.positions"].float()

  def forward(self, ctx):
    return ctx.ops.embed(self.tokens, ctx.token_ids, 1.0) + self.positions[ctx.positions.long()]


class UntiedHead(Head):
  """logits = x . W^T with a matrix of its own."""

  graph_safe = True

  def __init__(self, prefix, embedding, vocab_size, width):
    self.prefix, self.vocab_size, self.width = prefix, vocab_size, width

  def tensor_specs(self):
    return [TensorSpec(f"{self.prefix}.weight", (self.vocab_size, self.width), "matrix")]

  def bind(self, tensors, ops):
    self.weight = tensors[f"{self.prefix}.weight"]

  def forward(self, x, ctx):
    return ctx.ops.lm_head(x, self.weight, 0.0)


class DenselyRoutedFeedForward(FeedForward):
  """Soft routing without a look at the host: every expert acts on every token and the results
  are mixed with the router's softmax (float32 logits).  (The top-1 routing of the neighbouring
  test file jumps when bfloat16 rounding turns a near-tie of the router; a mixture does not.)"""

  graph_safe = True

  def __init__(self, prefix, width, hidden, experts):
    self.prefix, self.width, self.hidden, self.experts = prefix, width, hidden, experts

  def tensor_specs(self):
    specs = [TensorSpec(f"{self.prefix}.router.weight", (self.experts, self.width), "matrix", precision="stored")]
    for e in range(self.experts):
      specs += [TensorSpec(f"{self.prefix}.experts.{e}.gate_up.weight", (2 * self.hidden, self.width), "matrix"),
                TensorSpec(f"{self.prefix}.experts.{e}.down.weight", (self.width, self.hidden), "matrix")]
    return specs

  def bind(self, tensors, ops):
    self.router = tensors[f"{self.prefix}.router.weight"].float()
    self.gate_up = [tensors[f"{self.prefix}.experts.{e}.gate_up.weight"] for e in range(self.experts)]
    self.down = [tensors[f"{self.prefix}.experts.{e}.down.weight"] for e in range(self.experts)]

  def forward(self, x, ctx):
    ops = ctx.ops
    logits = x.float() @ self.router.t()
    prob = torch.softmax(logits, dim=-1)
    out = torch.zeros_like(x, dtype=torch.float32)
    for e in range(self.experts):
      y = ops.linear(ops.gated_linear(x, self.gate_up[e], 0), self.down[e]).float()
      out = out + y * prob[:, e:e + 1]
    return out.to(x.dtype)


@pytest.fixture(scope="module", autouse=True)
def registered():
  EMBEDDINGS.register("toy_positioned", PositionedEmbedding)
  HEADS.register("toy_untied", UntiedHead)
  FEED_FORWARDS.register("toy_dense_routed", DenselyRoutedFeedForward)
  yield
  EMBEDDINGS.unregister("toy_positioned")
  HEADS.unregister("toy_untied")
  FEED_FORWARDS.unregister("toy_dense_routed")


def toy_spec():
  norm = PartSpec("rms_norm", params={"eps": EPS, "plus_one": True})
  rotary = PartSpec("rotary", params={"theta": THETA, "scale_factor": 1.0})
  layers = []
  for name, (hq, hkv, dh) in LAYERS.items():
    attention = PartSpec("paged_attention", f"{name}.attn", dict(
        width=WIDTH, num_heads=hq, num_kv_heads=hkv, head_dim=dh, query_scale=dh ** -0.5, logit_softcap=CAP,
        window=None, position=rotary))
    routed = PartSpec("toy_dense_routed", f"{name}.moe", dict(width=WIDTH, hidden=HIDDEN, experts=EXPERTS))
    layers.append(LayerSpec(name, PartSpec("pre_norm", name, dict(width=WIDTH, norm=norm)), attention, routed))
  return ModelSpec(
      architecture="ToyGraphsForTests", vocab_size=VOCAB, width=WIDTH, max_context=MAX_POS,
      embedding=PartSpec("toy_positioned", "emb", dict(vocab_size=VOCAB, width=WIDTH, max_positions=MAX_POS)),
      layers=tuple(layers), run_order=(LayerCall("A"), LayerCall("B")),
      final_norm=PartSpec("rms_norm", "final", dict(width=WIDTH, eps=EPS, plus_one=True)),
      head=PartSpec("toy_untied", "out", dict(vocab_size=VOCAB, width=WIDTH)))


class ToyConfig:
  eos_token_id = None

  def model_spec(self):
    return toy_spec()


def plain_forward(t, tokens):
  f = lambda name: t[name].float().numpy()
  pos = np.arange(len(tokens))
  h = f("emb.tokens")[np.asarray(tokens)] + f("emb.positions")[pos]
  for name, (hq, hkv, dh) in LAYERS.items():
    y = plain.rms_norm(h, f(f"{name}.pre_mixer.weight"), EPS)
    q = plain.rope((y @ f(f"{name}.attn.q_proj.weight").T).reshape(-1, hq, dh), pos, THETA) * np.float32(dh ** -0.5)
    k = plain.rope((y @ f(f"{name}.attn.k_proj.weight").T).reshape(-1, hkv, dh), pos, THETA)
    v = (y @ f(f"{name}.attn.v_proj.weight").T).reshape(-1, hkv, dh)
    o = plain.grouped_attention(q, k, v, pos, pos, CAP, None)
    h = h + o.reshape(len(tokens), -1) @ f(f"{name}.attn.o_proj.weight").T
    y = plain.rms_norm(h, f(f"{name}.pre_feed_forward.weight"), EPS)
    logits = y @ f(f"{name}.moe.router.weight").T
    prob = np.exp(logits - logits.max(-1, keepdims=True))
    prob /= prob.sum(-1, keepdims=True)
    out = np.zeros_like(y)
    for e in range(EXPERTS):
      gu = f(f"{name}.moe.experts.{e}.gate_up.weight")
      z = plain.gated_feed_forward(y, gu[:HIDDEN], gu[HIDDEN:], f(f"{name}.moe.experts.{e}.down.weight"))
      out += z * prob[:, e:e + 1]
    h = h + out
  return plain.rms_norm(h, f("final.weight"), EPS) @ f("out.weight").T


def build(dtype, device, ops, **engine_kw):
  specs = DecoderModel(toy_spec()).tensor_specs()
  tensors = random_tensors(specs, 11, matrix_std=0.12, scale_std=0.1, dtype=torch.bfloat16)
  on_device = {k: v.to(device=device, dtype=getattr(torch, dtype)) for k, v in tensors.items()}
  ec = EngineConfig(activation_dtype=dtype, page_size=8, batch_size=3, max_seq_len=MAX_POS,
                    max_cache_tokens=3 * MAX_POS, **engine_kw)
  return Engine(ToyConfig(), on_device, ec, ops=ops, device=device), tensors


def test_registered_embedding_and_head_kinds_on_the_cpu_kernel_table():
  engine, tensors = build("float32", "cpu", ReferenceOps(torch.float32))
  assert type(engine.model.embedding) is PositionedEmbedding and type(engine.model.head) is UntiedHead
  assert engine.model.graph_safe()
  toks = np.random.default_rng(1).integers(0, VOCAB, 50).tolist()
  slot = engine.open_request()
  got = [engine.step_raw([StepEntry(slot, toks[:21], tuple(range(21)))])]
  got += [engine.step_raw([StepEntry(slot, [t], (0,))]) for t in toks[21:]]
  assert_logits_close(torch.cat(got).numpy(), plain_forward(tensors, toks), "float32", "cpu")


def test_an_unknown_kind_is_refused_by_name():
  import dataclasses
  bad = dataclasses.replace(toy_spec(), head=PartSpec("no_such_head", "out", {}))
  with pytest.raises(KeyError, match="head: unknown name 'no_such_head'"):
    DecoderModel(bad)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_foreign_graph_safe_parts_decode_from_cuda_graphs(dtype):
  engine, tensors = build(dtype, "cuda", None, intermediate_steps=5)
  runner = engine._decode_runner
  assert runner is not None  # every part is graph-safe, foreign or not
  runner.keep_logits = True
  # The two layers share (window, group) but not the head size: each has work lists of its own.
  keys = {p.key for p in runner._plans(2, 1024)}
  assert len(keys) == (2 if dtype == "bfloat16" else 0)
  rng = np.random.default_rng(2)
  prompts = [rng.integers(0, VOCAB, n).tolist() for n in (30, 77, 9)]
  bursts = []
  inner = engine._decode_burst

  def burst(plan):
    before = [(e.request, len(e.request.tokens) - 1) for e in plan.entries]
    finished = inner(plan)
    bursts.append((before, [len(r.tokens) for r, _ in before], runner.last_logits.float().cpu().numpy()))
    return finished

  engine._decode_burst = burst
  results = engine.generate(prompts, [SamplingParams(temperature=0.0, max_decode_steps=n, stop_token_ids=())
                                      for n in (40, 22, 31)])
  engine.ops.check_errors()
  assert bursts and max(b[2].shape[0] for b in bursts) == 5
  want = {r.request_id: plain_forward(tensors, (p + r.output_token_ids)[:-1]) for p, r in zip(prompts, results)}
  checked = 0
  for before, lengths_after, logits in bursts:
    for j, ((r, pos0), n_after) in enumerate(zip(before, lengths_after)):
      rows = [i for i in range(logits.shape[0]) if pos0 + i < n_after - 1]
      if rows:
        assert_logits_close(logits[rows, j], want[r.request_id][pos0:pos0 + len(rows)], dtype, "graph step")
        checked += len(rows)
  assert checked >= 80
  for p, r in zip(prompts, results):
    w = want[r.request_id]
    for i, tok in enumerate(r.output_token_ids):
      row = w[len(p) - 1 + i]
      bound = 2 * BF16_MAX * np.abs(w).max() if dtype == "bfloat16" else 1e-4 * np.abs(w).max()
      assert row.max() - row[tok] <= bound


@pytest.mark.gpu
def test_the_toy_routed_feed_forward_that_looks_at_the_host_still_runs_eagerly():
  """A part that does not say it is graph-safe keeps the model on eager steps."""
  class Unsafe(DenselyRoutedFeedForward):
    graph_safe = False

  FEED_FORWARDS.register("toy_dense_routed", Unsafe, replace=True)
  try:
    engine, _ = build("float32", "cuda", None)
    assert engine._decode_runner is None
  finally:
    FEED_FORWARDS.register("toy_dense_routed", DenselyRoutedFeedForward, replace=True)
