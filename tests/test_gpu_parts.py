"""Each part of a layer alone on the GPU, built from parameters only (no model around it),
against the plain NumPy function of the same part, in float32 and bfloat16."""

import numpy as np
import pytest
import torch

from simply_b200.cache import CacheManager
from simply_b200.config.model_spec import PartSpec
from simply_b200.engine.batch import StepEntry, pack_step
from simply_b200.parts.attention import PagedAttention
from simply_b200.parts.block import PreNormBlock, ResidualStream, SandwichNormBlock
from simply_b200.parts.embedding import TiedHead, TokenEmbedding
from simply_b200.parts.feedforward import GatedFeedForward
from simply_b200.parts.norm import RMSNorm
from simply_b200.parts.position import NoPositionEncoding, RotaryEncoding
from simply_b200.weights import random_tensors
from tests.plain import gemma2_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
WIDTH, HQ, HKV, DH, FFN, VOCAB = 72, 6, 3, 48, 200, 333


@pytest.fixture(scope="module")
def tables():
  from simply_b200.kernels.ops import CudaOps
  return {"float32": CudaOps(torch.float32), "bfloat16": CudaOps(torch.bfloat16)}


def bound(part, dtype, ops, seed=0, scale_std=0.3):
  t = random_tensors(part.tensor_specs(), seed, matrix_std=0.1, scale_std=scale_std, dtype=torch.bfloat16)
  part.bind({k: v.to("cuda", getattr(torch, dtype)) for k, v in t.items()}, ops)
  return {k: v.float().numpy() for k, v in t.items()}


def context(ops, need, lengths, page=8, dtype="float32"):
  """A step that brings `lengths[i]` first tokens of request i (no history)."""
  mgr = CacheManager({"c": need} if need is not None else {}, page_size=page, max_slots=len(lengths),
                     max_seq_len=128, max_cache_tokens=128 * len(lengths), dtype=getattr(torch, dtype), device="cuda")
  slots = [mgr.acquire_slot(i) for i in range(len(lengths))]
  entries = [StepEntry(s, [0] * n, ()) for s, n in zip(slots, lengths)]
  mgr.extend([(s, n) for s, n in zip(slots, lengths)])
  ctx = pack_step(entries, [0] * len(lengths), [g.tables for g in mgr.groups], page, ops, "cuda")
  return mgr, ctx


def close(got, want, dtype, scale=None):
  got = got.float().cpu().numpy()
  scale = scale or max(np.abs(want).max(), 1e-6)
  bound_ = 2e-5 if dtype == "float32" else 2e-2
  assert np.abs(got - want).max() <= bound_ * scale, (np.abs(got - want).max(), scale)


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(tables, dtype):
  ops = tables[dtype]
  for plus_one, eps in ((True, 1e-6), (False, 1e-3)):
    n = RMSNorm("n", WIDTH, eps, plus_one)
    w = bound(n, dtype, ops)
    x = torch.randn(9, WIDTH) * 4
    _, ctx = context(ops, None, [9])
    close(n.apply(x.cuda(), ctx), plain.rms_norm(x.numpy(), w["n.weight"], eps, plus_one), dtype)


@pytest.mark.parametrize("theta", [10000.0, 77.0])
def test_position_part(tables, theta):
  ops = tables["float32"]
  _, ctx = context(ops, None, [5, 3])
  cos, sin = RotaryEncoding(theta=theta).rotation_tables(ctx, DH)
  x = np.random.default_rng(0).normal(size=(8, 2, DH)).astype(np.float32)
  pos = ctx.host["positions"]
  half = DH // 2
  c, s = cos.cpu().numpy()[:, None, :], sin.cpu().numpy()[:, None, :]
  rotated = np.concatenate([x[..., :half] * c - x[..., half:] * s, x[..., half:] * c + x[..., :half] * s], -1)
  np.testing.assert_allclose(rotated, plain.rope(x, pos, theta), atol=1e-5)
  assert pos.tolist() == [0, 1, 2, 3, 4, 0, 1, 2]
  assert NoPositionEncoding().rotation_tables(ctx, DH) is None
  # computed once per step and parameter set, then shared by all layers
  assert RotaryEncoding(theta=theta).rotation_tables(ctx, DH)[0].data_ptr() == cos.data_ptr()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,cap,rotary", [(None, 30.0, True), (5, 0.0, True), (7, 50.0, False)])
def test_attention_part(tables, dtype, window, cap, rotary):
  ops = tables[dtype]
  pos_spec = PartSpec("rotary", params={"theta": 500.0}) if rotary else None
  mixer = PagedAttention("a", WIDTH, HQ, HKV, DH, query_scale=0.25, logit_softcap=cap, window=window,
                         position=pos_spec)
  w = bound(mixer, dtype, ops)
  lengths = [19, 1, 8]
  mgr, ctx = context(ops, mixer.cache_need(), lengths, dtype=dtype)
  x = (torch.randn(sum(lengths), WIDTH) * 1.5).to(getattr(torch, dtype))
  got = mixer.forward(x.cuda(), ctx, mgr.paged["c"])
  ops.check_errors()
  cfg = dict(num_attention_heads=HQ, num_key_value_heads=HKV, head_dim=DH, rope_theta=500.0,
             query_pre_attn_scalar=16.0, attn_logit_softcapping=cap, sliding_window=window or 10 ** 6,
             layer_types=["sliding_attention"])
  ww = {k: w[f"a.{k}_proj.weight"] for k in "qkvo"}
  r = 0
  for n in lengths:
    xs = x[r:r + n].float().numpy()
    if rotary:
      want, _ = plain.attention_layer(xs, np.arange(n), ww, cfg, 0)
    else:  # no rotation: the plain function with a rotary base that turns nothing is not available, so by hand
      q = (xs @ ww["q"].T).reshape(n, HQ, DH) * 0.25
      k, v = (xs @ ww["k"].T).reshape(n, HKV, DH), (xs @ ww["v"].T).reshape(n, HKV, DH)
      o = plain.grouped_attention(q, k, v, np.arange(n), np.arange(n), cap, window)
      want = o.reshape(n, HQ * DH) @ ww["o"].T
    close(got[r:r + n], want, dtype, np.abs(want).max())
    r += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens", [3, 40])
def test_feed_forward_part(tables, dtype, tokens):
  ops = tables[dtype]
  ffn = GatedFeedForward("f", WIDTH, FFN, "gelu_tanh")
  w = bound(ffn, dtype, ops)
  x = (torch.randn(tokens, WIDTH) * 2).to(getattr(torch, dtype))
  _, ctx = context(ops, None, [tokens])
  want = plain.gated_feed_forward(x.float().numpy(), w["f.gate_proj.weight"], w["f.up_proj.weight"], w["f.down_proj.weight"])
  close(ffn.forward(x.cuda(), ctx), want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["sandwich_norm", "pre_norm"])
def test_block_part(tables, dtype, kind):
  ops = tables[dtype]
  mixer = PagedAttention("b.attn", WIDTH, HQ, HKV, DH, query_scale=0.2, logit_softcap=20.0, window=6,
                         position=PartSpec("rotary", params={"theta": 1000.0}))
  ffn = GatedFeedForward("b.ffn", WIDTH, FFN, "gelu_tanh")
  cls = SandwichNormBlock if kind == "sandwich_norm" else PreNormBlock
  block = cls("b", WIDTH, PartSpec("rms_norm", params={"eps": 1e-5, "plus_one": True}), mixer, ffn)
  w = bound(block, dtype, ops)
  n = 23
  mgr, ctx = context(ops, block.cache_need(), [n], dtype=dtype)
  h0 = torch.randn(n, WIDTH) * 3
  stream = ResidualStream(h0.clone().cuda())
  block.forward(stream, ctx, mgr.paged["c"])
  stream.flush(ctx)
  cfg = dict(num_attention_heads=HQ, num_key_value_heads=HKV, head_dim=DH, rope_theta=1000.0,
             query_pre_attn_scalar=25.0, attn_logit_softcapping=20.0, sliding_window=6,
             layer_types=["sliding_attention"])
  ww = {k: w[f"b.attn.{k}_proj.weight"] for k in "qkvo"}
  h = h0.numpy()
  a, _ = plain.attention_layer(plain.rms_norm(h, w["b.pre_mixer.weight"], 1e-5), np.arange(n), ww, cfg, 0)
  h = h + (plain.rms_norm(a, w["b.post_mixer.weight"], 1e-5) if kind == "sandwich_norm" else a)
  f = plain.gated_feed_forward(plain.rms_norm(h, w["b.pre_feed_forward.weight"], 1e-5), w["b.ffn.gate_proj.weight"],
                               w["b.ffn.up_proj.weight"], w["b.ffn.down_proj.weight"])
  h = h + (plain.rms_norm(f, w["b.post_feed_forward.weight"], 1e-5) if kind == "sandwich_norm" else f)
  assert stream.h.dtype == torch.float32  # the residual stream stays in 32 bits
  close(stream.h, h, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(tables, dtype):
  ops = tables[dtype]
  emb = TokenEmbedding("e", VOCAB, WIDTH, scale=WIDTH ** 0.5)
  head = TiedHead("e", emb, logit_softcap=15.0)
  w = bound(emb, dtype, ops)
  _, ctx = context(ops, None, [6])
  ids = torch.tensor([0, 5, 332, 7, 7, 100], dtype=torch.int32)
  ctx.token_ids.copy_(ids)
  scale = float(torch.tensor(WIDTH ** 0.5).to(getattr(torch, dtype)))
  close(emb.forward(ctx), w["e.weight"][ids.long().numpy()] * scale, dtype)
  x = (torch.randn(4, WIDTH) * 3).to(getattr(torch, dtype))
  logits = head.forward(x.cuda(), ctx)
  assert logits.dtype == torch.float32
  want = plain.soft_cap(x.float().numpy() @ w["e.weight"].T, 15.0)
  np.testing.assert_allclose(logits.cpu().numpy(), want, atol=2e-4, rtol=1e-4)  # float32 product in both dtypes
