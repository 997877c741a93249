"""Generality of the parts, continued: a toy model, defined here and nowhere in the package, with

  * a feed-forward with routing: every token goes to the one of E small gated feed-forwards that
    its router scores highest (router logits in float32), weighted by the router's softmax, and
  * another position encoding: only the first `rotary_dims` dims of a head rotate (the rest keep
    cos = 1, sin = 0), with positions counted from an offset,

both registered by this file through the public registries and built from a hand-written
ModelSpec, without a change to the package.  Logits are compared with a composition of the plain
NumPy functions, whole and in portions mixed with another request.  A test fixture, not a model
of anyone's."""

import numpy as np
import pytest
import torch

from simply_b200 import Engine, EngineConfig, StepEntry
from simply_b200.config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from simply_b200.parts.base import FeedForward, PositionEncoding
from simply_b200.parts.model import DecoderModel
from simply_b200.registry import FEED_FORWARDS, POSITION_ENCODINGS
from simply_b200.weights import TensorSpec, random_tensors
from tests.plain import gemma2_plain as plain
from tests.reference_ops import ReferenceOps
from tests.tolerances import assert_logits_close

WIDTH, VOCAB, HQ, HKV, DH, HIDDEN, EXPERTS = 40, 157, 6, 3, 32, 24, 3
EPS, THETA, QSCALE, CAP, FINAL_CAP, ROTARY_DIMS, OFFSET = 1e-6, 100.0, 0.25, 0.0, 0.0, 16, 3


class RoutedFeedForward(FeedForward):
  """Top-1 routing over `experts` gated feed-forwards; the products go through the kernel table,
  the routing itself is a few tensor operations of the test."""

  def __init__(self, prefix, width, hidden, experts):
    self.prefix, self.width, self.hidden, self.experts = prefix, width, hidden, experts

  def tensor_specs(self):
    specs = [TensorSpec(f"{self.prefix}.router.weight", (self.experts, self.width), "matrix")]
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
    logits = x.float() @ self.router.t()  # float32 router logits
    prob = torch.softmax(logits, dim=-1)
    choice = torch.argmax(logits, dim=-1)
    out = torch.zeros_like(x)
    for e in range(self.experts):
      rows = torch.nonzero(choice == e).flatten()
      if rows.numel() == 0:
        continue
      y = ops.linear(ops.gated_linear(x[rows].contiguous(), self.gate_up[e], 0), self.down[e])
      out[rows] = (y.float() * prob[rows, e:e + 1]).to(x.dtype)
    return out


class PartialRotary(PositionEncoding):
  """The first `rotary_dims` dims of a head rotate with angle (position + offset) / timescale;
  the others stay as they are.  Pairs are (j, j + head_dim / 2) as everywhere in the engine."""

  def __init__(self, prefix="", theta=10000.0, rotary_dims=0, offset=0):
    self.theta, self.rotary_dims, self.offset = float(theta), int(rotary_dims), int(offset)

  def rotation_tables(self, ctx, head_dim):
    key = ("partial_rotary", self.theta, self.rotary_dims, self.offset, head_dim)
    tables = ctx.memo.get(key)
    if tables is None:
      half, rot = head_dim // 2, self.rotary_dims // 2
      j = torch.arange(half, device=ctx.positions.device, dtype=torch.float32)
      timescale = torch.pow(torch.tensor(self.theta, device=j.device), 2 * j / self.rotary_dims)
      angle = (ctx.positions.float()[:, None] + self.offset) / timescale[None, :]
      angle = torch.where(j[None, :] < rot, angle, torch.zeros_like(angle))
      tables = ctx.memo[key] = (torch.cos(angle).contiguous(), torch.sin(angle).contiguous())
    return tables


@pytest.fixture(scope="module", autouse=True)
def registered():
  FEED_FORWARDS.register("toy_routed", RoutedFeedForward)
  POSITION_ENCODINGS.register("toy_partial_rotary", PartialRotary)
  yield
  FEED_FORWARDS.unregister("toy_routed")
  POSITION_ENCODINGS.unregister("toy_partial_rotary")


def toy_spec():
  norm = PartSpec("rms_norm", params={"eps": EPS, "plus_one": False})
  position = PartSpec("toy_partial_rotary", params={"theta": THETA, "rotary_dims": ROTARY_DIMS, "offset": OFFSET})

  def layer(name, window):
    attention = PartSpec("paged_attention", f"{name}.attn", dict(
        width=WIDTH, num_heads=HQ, num_kv_heads=HKV, head_dim=DH, query_scale=QSCALE, logit_softcap=CAP,
        window=window, position=position))
    routed = PartSpec("toy_routed", f"{name}.moe", dict(width=WIDTH, hidden=HIDDEN, experts=EXPERTS))
    return LayerSpec(name, PartSpec("pre_norm", name, dict(width=WIDTH, norm=norm)), attention, routed)

  layers = (layer("A", None), layer("B", 9))
  return ModelSpec(
      architecture="ToyRoutedForTests", vocab_size=VOCAB, width=WIDTH, max_context=128,
      embedding=PartSpec("token_embedding", "emb", dict(vocab_size=VOCAB, width=WIDTH, scale=1.0)),
      layers=layers, run_order=(LayerCall("A"), LayerCall("B")),
      final_norm=PartSpec("rms_norm", "final", dict(width=WIDTH, eps=EPS, plus_one=False)),
      head=PartSpec("tied_head", "emb", dict(logit_softcap=FINAL_CAP)))


class ToyConfig:
  eos_token_id = None

  def model_spec(self):
    return toy_spec()


def plain_partial_rope(x, positions):
  """x [T, H, dh]: rotation of the first ROTARY_DIMS dims, pairs (j, j + dh/2), from the plain rope's formula."""
  half, rot = DH // 2, ROTARY_DIMS // 2
  j = np.arange(half, dtype=np.float32)
  timescale = np.power(np.float32(THETA), 2 * j / ROTARY_DIMS).astype(np.float32)
  angle = (positions.astype(np.float32)[:, None] + OFFSET) / timescale[None, :]
  angle = np.where(j[None, :] < rot, angle, 0.0).astype(np.float32)
  c, s = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
  x1, x2 = x[..., :half], x[..., half:]
  return np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], axis=-1)


def plain_forward(t, tokens):
  f = lambda name: t[name].float().numpy()
  pos = np.arange(len(tokens))
  h = f("emb.weight")[np.asarray(tokens)]

  def rms(x, name):
    return plain.rms_norm(x, f(name), EPS, plus_one=False)

  for name, window in (("A", None), ("B", 9)):
    y = rms(h, f"{name}.pre_mixer.weight")
    q = (y @ f(f"{name}.attn.q_proj.weight").T).reshape(-1, HQ, DH)
    k = (y @ f(f"{name}.attn.k_proj.weight").T).reshape(-1, HKV, DH)
    v = (y @ f(f"{name}.attn.v_proj.weight").T).reshape(-1, HKV, DH)
    q, k = plain_partial_rope(q, pos) * np.float32(QSCALE), plain_partial_rope(k, pos)
    o = plain.grouped_attention(q, k, v, pos, pos, CAP, window)
    h = h + o.reshape(len(tokens), -1) @ f(f"{name}.attn.o_proj.weight").T
    y = rms(h, f"{name}.pre_feed_forward.weight")
    logits = y @ f(f"{name}.moe.router.weight").T
    prob = np.exp(logits - logits.max(-1, keepdims=True))
    prob /= prob.sum(-1, keepdims=True)
    out = np.zeros_like(y)
    for i, e in enumerate(np.argmax(logits, -1)):
      gu = f(f"{name}.moe.experts.{e}.gate_up.weight")
      z = plain.gated_feed_forward(y[i:i + 1], gu[:HIDDEN], gu[HIDDEN:], f(f"{name}.moe.experts.{e}.down.weight"))
      out[i] = z[0] * prob[i, e]
    h = h + out
  x = rms(h, "final.weight")
  return x @ f("emb.weight").T


def build(dtype, device, ops):
  specs = DecoderModel(toy_spec()).tensor_specs()
  tensors = random_tensors(specs, 3, matrix_std=0.15, scale_std=0.2, dtype=torch.bfloat16)
  on_device = {k: v.to(device=device, dtype=getattr(torch, dtype)) for k, v in tensors.items()}
  ec = EngineConfig(activation_dtype=dtype, page_size=8, batch_size=2, max_seq_len=128, max_cache_tokens=128)
  return Engine(ToyConfig(), on_device, ec, ops=ops, device=device), tensors


def check(engine, tensors, dtype):
  rng = np.random.default_rng(8)
  reqs = [rng.integers(0, VOCAB, n).tolist() for n in (29, 17)]
  want = [plain_forward(tensors, r) for r in reqs]
  for toks, w in zip(reqs, want):
    slot = engine.open_request()
    got = engine.step_raw([StepEntry(slot, toks, tuple(range(len(toks))))])
    assert_logits_close(got.float().cpu().numpy(), w, dtype, "whole")
    engine.close_request(slot)
  # portions of one request beside single tokens of the other
  slots = [engine.open_request() for _ in reqs]
  got = [[] for _ in reqs]
  pos = [0, 0]
  sizes = [4, 2, 9, 3]
  step = 0
  while any(p < len(r) for p, r in zip(pos, reqs)):
    entries, who = [], []
    for i, toks in enumerate(reqs):
      if pos[i] >= len(toks):
        continue
      n = 1 if i == 1 else min(sizes[step % len(sizes)], len(toks) - pos[i])
      entries.append(StepEntry(slots[i], toks[pos[i]:pos[i] + n], tuple(range(n))))
      who.append((i, n))
      pos[i] += n
    step += 1
    logits = engine.step_raw(entries).float().cpu().numpy()
    r = 0
    for i, n in who:
      got[i].append(logits[r:r + n])
      r += n
  for g, w in zip(got, want):
    assert_logits_close(np.concatenate(g), w, dtype, "portions")
  engine.cache.check_invariants()


def test_routed_feed_forward_and_partial_rotary_on_the_cpu_kernel_table():
  engine, tensors = build("float32", "cpu", ReferenceOps(torch.float32))
  check(engine, tensors, "float32")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_and_partial_rotary_on_the_gpu(dtype):
  engine, tensors = build(dtype, "cuda", None)
  assert engine._decode_runner is None  # foreign parts: steps run eagerly, not from a graph
  check(engine, tensors, dtype)
  engine.ops.check_errors()
