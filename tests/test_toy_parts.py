"""Generality of the parts: a toy model, defined here and nowhere in the package, that

  * runs one layer twice (same weights, a cache per call),
  * lets a layer without k/v projections read the cache another call wrote,
  * uses a mixer with per-request state of fixed size (a running mean), registered here,
  * mixes block arrangements (sandwich norms, pre-norm only) and window / no window,

is built from a hand-written ModelSpec, stepped whole, in portions and mixed with other
requests, and compared with a composition of the plain NumPy functions.  It is a test
fixture, not a model of anyone's."""

import numpy as np
import pytest
import torch

from simply_b200 import Engine, EngineConfig, StepEntry
from simply_b200.cache import SlotStateNeed
from simply_b200.config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from simply_b200.parts.base import Mixer
from simply_b200.parts.model import DecoderModel
from simply_b200.registry import MIXERS
from simply_b200.weights import TensorSpec, random_tensors
from tests.plain import gemma2_plain as plain
from tests.reference_ops import ReferenceOps
from tests.tolerances import assert_logits_close

WIDTH, VOCAB, HQ, HKV, DH, FFN, WINDOW = 48, 211, 4, 2, 16, 80, 6
EPS, THETA, QSCALE, CAP, FINAL_CAP = 1e-5, 1000.0, 0.3, 30.0, 20.0


class RunningMeanMixer(Mixer):
  """y[t] = gain * mean(x[0..t]) over the request's tokens; the state (sum, count) lives in the
  request's slot, so a request may arrive in any portions."""

  def __init__(self, prefix, width):
    self.prefix, self.width = prefix, width
    self.gain = None

  def cache_need(self):
    return SlotStateNeed((self.width + 1,), "float32")

  def tensor_specs(self):
    return [TensorSpec(f"{self.prefix}.gain", (self.width,), "scale")]

  def bind(self, tensors, ops):
    self.gain = tensors[f"{self.prefix}.gain"].float()

  def forward(self, x, ctx, cache, writes_cache=True):
    out = torch.empty_like(x)
    cu_q, slots = ctx.host["cu_q"], ctx.host["slots"]
    for b in range(ctx.num_seqs):
      r0, r1 = int(cu_q[b]), int(cu_q[b + 1])
      state = cache.storage[int(slots[b])]
      sums = state[:self.width] + torch.cumsum(x[r0:r1].float(), dim=0)
      counts = state[self.width] + torch.arange(1, r1 - r0 + 1, device=x.device, dtype=torch.float32)
      out[r0:r1] = (sums / counts[:, None] * (1.0 + self.gain)).to(x.dtype)
      state[:self.width] = sums[-1]
      state[self.width] = counts[-1]
    return out


@pytest.fixture(scope="module", autouse=True)
def registered():
  MIXERS.register("toy_running_mean", RunningMeanMixer)
  yield
  MIXERS.unregister("toy_running_mean")


def toy_spec():
  norm = PartSpec("rms_norm", params={"eps": EPS, "plus_one": True})
  rotary = PartSpec("rotary", params={"theta": THETA, "scale_factor": 1.0})

  def attention(prefix, window, project_kv=True):
    return PartSpec("paged_attention", prefix, dict(
        width=WIDTH, num_heads=HQ, num_kv_heads=HKV, head_dim=DH, query_scale=QSCALE, logit_softcap=CAP,
        window=window, position=rotary, project_kv=project_kv))

  def ffn(prefix):
    return PartSpec("gated", prefix, dict(width=WIDTH, hidden=FFN, activation="gelu_tanh"))

  layers = (
      LayerSpec("L0", PartSpec("sandwich_norm", "L0", dict(width=WIDTH, norm=norm)), attention("L0.attn", WINDOW), ffn("L0.ffn")),
      LayerSpec("L1", PartSpec("pre_norm", "L1", dict(width=WIDTH, norm=norm)),
                PartSpec("toy_running_mean", "L1.mix", dict(width=WIDTH)), ffn("L1.ffn")),
      LayerSpec("L2", PartSpec("sandwich_norm", "L2", dict(width=WIDTH, norm=norm)),
                attention("L2.attn", WINDOW - 2, project_kv=False), ffn("L2.ffn")),
  )
  order = (LayerCall("L0"), LayerCall("L1"), LayerCall("L0"), LayerCall("L2", cache="L0#0", writes_cache=False))
  return ModelSpec(
      architecture="ToyForTests", vocab_size=VOCAB, width=WIDTH, max_context=256,
      embedding=PartSpec("token_embedding", "emb", dict(vocab_size=VOCAB, width=WIDTH, scale=WIDTH ** 0.5)),
      layers=layers, run_order=order, final_norm=PartSpec("rms_norm", "final", dict(width=WIDTH, eps=EPS)),
      head=PartSpec("tied_head", "emb", dict(logit_softcap=FINAL_CAP)))


class ToyConfig:
  eos_token_id = None

  def model_spec(self):
    return toy_spec()


def plain_forward(t, tokens):
  """The toy model from the plain functions (float32 NumPy, whole sequence, no cache)."""
  f = lambda name: t[name].float().numpy()
  pos = np.arange(len(tokens))
  cfg = dict(num_attention_heads=HQ, num_key_value_heads=HKV, head_dim=DH, rope_theta=THETA,
             query_pre_attn_scalar=QSCALE ** -2, attn_logit_softcapping=CAP, sliding_window=WINDOW)

  def attn(y, prefix, window, k_override=None):
    w = {"q": f(f"{prefix}.q_proj.weight"), "o": f(f"{prefix}.o_proj.weight")}
    if k_override is None:
      w["k"], w["v"] = f(f"{prefix}.k_proj.weight"), f(f"{prefix}.v_proj.weight")
    return plain.attention_layer(y, pos, w, dict(cfg, sliding_window=window, layer_types=["sliding_attention"]),
                                 0, k_override)

  def ffn(y, prefix):
    return plain.gated_feed_forward(y, f(f"{prefix}.gate_proj.weight"), f(f"{prefix}.up_proj.weight"),
                                    f(f"{prefix}.down_proj.weight"))

  def sandwich(h, name, window, k_override=None):
    a, kv = attn(plain.rms_norm(h, f(f"{name}.pre_mixer.weight"), EPS), f"{name}.attn", window, k_override)
    h = h + plain.rms_norm(a, f(f"{name}.post_mixer.weight"), EPS)
    g = ffn(plain.rms_norm(h, f(f"{name}.pre_feed_forward.weight"), EPS), f"{name}.ffn")
    return h + plain.rms_norm(g, f(f"{name}.post_feed_forward.weight"), EPS), kv

  h = plain.embed(tokens, f("emb.weight"))
  h, kv0 = sandwich(h, "L0", WINDOW)
  y = plain.rms_norm(h, f("L1.pre_mixer.weight"), EPS)
  mean = np.cumsum(y, axis=0) / np.arange(1, len(tokens) + 1, dtype=np.float32)[:, None]
  h = h + mean * (1.0 + f("L1.mix.gain"))
  h = h + ffn(plain.rms_norm(h, f("L1.pre_feed_forward.weight"), EPS), "L1.ffn")
  h, _ = sandwich(h, "L0", WINDOW)
  h, _ = sandwich(h, "L2", WINDOW - 2, k_override=kv0)  # a narrower window over the cache L0's first call wrote
  cfg_head = dict(rms_norm_eps=EPS, final_logit_softcapping=FINAL_CAP)
  return plain.logits_from_hidden(h, f("final.weight"), f("emb.weight"), cfg_head)


def build(dtype, device, ops):
  spec = toy_spec()
  specs = DecoderModel(spec).tensor_specs()
  assert "L2.attn.k_proj.weight" not in [s.name for s in specs]  # the reading layer has no k/v weights
  tensors = random_tensors(specs, 11, matrix_std=0.08, scale_std=0.2, dtype=torch.bfloat16)
  on_device = {k: v.to(device=device, dtype=getattr(torch, dtype)) for k, v in tensors.items()}
  ec = EngineConfig(activation_dtype=dtype, page_size=4, batch_size=3, max_seq_len=128, max_cache_tokens=160)
  return Engine(ToyConfig(), on_device, ec, ops=ops, device=device), tensors


def check(engine, tensors, dtype):
  assert engine.model.cache_names == ["L0#0", "L1#1", "L0#2", "L0#0"]
  assert set(engine.cache.paged) == {"L0#0", "L0#2"} and set(engine.cache.states) == {"L1#1"}
  rng = np.random.default_rng(5)
  reqs = [rng.integers(0, VOCAB, n).tolist() for n in (37, 21, 50)]
  want = [plain_forward(tensors, r) for r in reqs]
  # whole
  for toks, w in zip(reqs, want):
    slot = engine.open_request()
    got = engine.step_raw([StepEntry(slot, toks, tuple(range(len(toks))))])
    assert_logits_close(got.float().cpu().numpy(), w, dtype, "whole")
    engine.close_request(slot)
  # portions of changing size, three requests side by side, each finishing at another time
  slots = [engine.open_request() for _ in reqs]
  pos = [0, 0, 0]
  got = [[] for _ in reqs]
  sizes = [5, 2, 7, 1, 3, 1, 1, 9, 2, 1]
  step = 0
  while any(p < len(r) for p, r in zip(pos, reqs)):
    entries, who = [], []
    for i, toks in enumerate(reqs):
      if pos[i] >= len(toks) or (step + i) % 4 == 3:
        continue
      n = min(sizes[(step + 2 * i) % len(sizes)], len(toks) - pos[i])
      entries.append(StepEntry(slots[i], toks[pos[i]:pos[i] + n], tuple(range(n))))
      who.append((i, n))
      pos[i] += n
    step += 1
    if not entries:
      continue
    logits = engine.step_raw(entries).float().cpu().numpy()
    r = 0
    for i, n in who:
      got[i].append(logits[r:r + n])
      r += n
  for g, w in zip(got, want):
    assert_logits_close(np.concatenate(g), w, dtype, "portions")
  for s in slots:
    engine.close_request(s)
  engine.cache.check_invariants()
  # the slot's state starts from zero for the next request
  slot = engine.open_request()
  got = engine.step_raw([StepEntry(slot, reqs[1], tuple(range(len(reqs[1]))))])
  assert_logits_close(got.float().cpu().numpy(), want[1], dtype, "slot reuse")


def test_toy_model_on_the_cpu_kernel_table():
  engine, tensors = build("float32", "cpu", ReferenceOps(torch.float32))
  check(engine, tensors, "float32")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_model_on_the_gpu(dtype):
  engine, tensors = build(dtype, "cuda", None)
  assert engine._decode_runner is None  # a foreign mixer: steps run eagerly
  check(engine, tensors, dtype)
  engine.ops.check_errors()


def test_a_reader_must_come_after_its_writer():
  spec = toy_spec()
  import dataclasses
  bad = dataclasses.replace(spec, run_order=(LayerCall("L2", cache="L0#0", writes_cache=False),) + spec.run_order[:3])
  with pytest.raises(ValueError, match="no earlier call writes"):
    bad.validate()
  with pytest.raises(KeyError, match="does not define"):
    dataclasses.replace(spec, run_order=(LayerCall("nope"),)).validate()
  # a reader may not want more keys than the writer's cache keeps
  wide = dataclasses.replace(spec.layers[2], mixer=dataclasses.replace(
      spec.layers[2].mixer, params=dict(spec.layers[2].mixer.params, window=None)))
  with pytest.raises(ValueError, match="keeps only a window"):
    DecoderModel(dataclasses.replace(spec, layers=spec.layers[:2] + (wide,))).cache_needs()
