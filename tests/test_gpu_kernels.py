"""Each CUDA kernel alone against its plain PyTorch statement (tests/reference_ops.py),
at sizes other than the tiny models': widths and vocabularies that are no power of
two, head sizes in steps of 16, odd head counts and groups, several page sizes."""

import math
import types

import numpy as np
import pytest
import torch

from tests.kernel_util import make_scenario
from tests.plain import gemma2_plain as plain
from tests.reference_ops import ReferenceOps

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]


@pytest.fixture(scope="module")
def table():
  from simply_b200.kernels.ops import CudaOps
  return {dt: CudaOps(dt) for dt in DTYPES}


def tol(dtype, scale=1.0):
  # float32: sums in a different order; bfloat16: one rounding of the result (2^-9 relative)
  # on top of float32 arithmetic inside.
  return dict(atol=2e-5 * scale, rtol=2e-5) if dtype == torch.float32 else dict(atol=1e-2 * scale, rtol=1e-2)


def close(got, want, dtype, scale=1.0):
  torch.testing.assert_close(got.float().cpu(), want.float().cpu(), **tol(dtype, scale))


def norm_part(width, dtype, plus_one=True, eps=1e-6, seed=0, device="cuda"):
  g = torch.Generator().manual_seed(seed)
  w = (torch.randn(width, generator=g) * 0.3).to(dtype).to(device)
  return types.SimpleNamespace(weight=w, eps=eps, plus_one=plus_one)


# ---- embedding ---------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_embed(table, dtype):
  ops, ref = table[dtype], ReferenceOps(dtype)
  vocab, width = 1003, 72
  t = torch.randn(vocab, width).to(dtype).cuda()
  ids = torch.randint(0, vocab, (37,), dtype=torch.int32).cuda()
  got = ops.embed(t, ids, math.sqrt(width))
  assert got.dtype == torch.float32
  torch.testing.assert_close(got.cpu(), ref.embed(t.cpu(), ids.cpu(), math.sqrt(width)), atol=1e-6, rtol=1e-6)
  ops.check_errors()


# ---- norms --------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("width", [72, 2304, 3000])
@pytest.mark.parametrize("variant", ["pre_only", "post_pre", "add_only", "post_only", "rows"])
@pytest.mark.parametrize("rows_total", [19, 150])  # a block per row; a warp per row
def test_residual_norm(table, dtype, width, variant, rows_total):
  ops, ref = table[dtype], ReferenceOps(dtype)
  h = torch.randn(rows_total, width) * 3
  branch = (torch.randn(rows_total, width) * 2).to(dtype)
  post = norm_part(width, dtype, True, 1e-6, 1)
  pre = norm_part(width, torch.float32 if variant == "post_pre" else dtype, variant != "post_only", 1e-5, 2)
  rows = None
  if variant == "pre_only":
    args = (None, None, pre)
  elif variant == "post_pre":
    args = (branch, post, pre)
  elif variant == "add_only":
    args = (branch, None, pre)
  elif variant == "post_only":
    args = (branch, post, None)
  else:
    args = (branch, post, pre)
    rows = torch.tensor([18, 0, 7, 7] if rows_total < 64 else [149, 0, 7, 7] + list(range(20, 100)), dtype=torch.int32)

  def cpu(p):
    return None if p is None else types.SimpleNamespace(weight=p.weight.cpu(), eps=p.eps, plus_one=p.plus_one)

  h_ref = h.clone()
  want = ref.residual_norm(h_ref, None if args[0] is None else args[0].clone(), cpu(args[1]), cpu(args[2]), rows)
  h_dev = h.cuda()
  got = ops.residual_norm(h_dev, None if args[0] is None else args[0].cuda(), args[1], args[2],
                          None if rows is None else rows.cuda())
  if want is None:
    assert got is None
  else:
    close(got, want, dtype, scale=3.0)
  if rows is None:
    torch.testing.assert_close(h_dev.cpu(), h_ref, atol=1e-5, rtol=1e-5)
  else:
    torch.testing.assert_close(h_dev.cpu(), h)  # untouched when rows are gathered
  ops.check_errors()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_rms_norm_and_helpers(table, dtype):
  ops, ref = table[dtype], ReferenceOps(dtype)
  x = torch.randn(11, 200)
  n = norm_part(200, dtype, False, 1e-5)
  for xin in (x, x.to(dtype)):
    close(ops.rms_norm(xin.cuda(), n.weight, n.eps, n.plus_one), ref.rms_norm(xin, n.weight.cpu(), n.eps, n.plus_one), dtype, 3.0)
  rows = torch.tensor([3, 3, 10, 0], dtype=torch.int32)
  assert torch.equal(ops.gather_rows(x.cuda(), rows.cuda()).cpu(), x[rows.long()])
  h = x.clone().cuda()
  ops.add_to_residual(h, x.to(dtype).cuda())
  torch.testing.assert_close(h.cpu(), x + x.to(dtype).float())


# ---- rotation and cache write ----------------------------------------------------
@pytest.mark.parametrize("theta,half", [(10000.0, 8), (500000.0, 24), (10000.0, 128)])
def test_rotation_tables(table, theta, half):
  ops, ref = table[torch.float32], ReferenceOps(torch.float32)
  pos = torch.tensor([0, 1, 2, 63, 64, 1000, 8191, 40000], dtype=torch.int32)
  frac = (2 * np.arange(half) / (2 * half)).astype(np.float32)
  ts = torch.from_numpy(np.power(np.float32(theta), frac).astype(np.float32))
  cos, sin = ops.rotation_tables(pos.cuda(), ts.cuda(), 1.0)
  rc, rs = ref.rotation_tables(pos, ts, 1.0)
  # Same float32 angle on both sides; sin/cos implementations differ by a few ulp.
  torch.testing.assert_close(cos.cpu(), rc, atol=2e-6, rtol=0)
  torch.testing.assert_close(sin.cpu(), rs, atol=2e-6, rtol=0)
  # Against float64 angles the float32 angle itself is off by up to pos * 2^-24.
  exact = pos.double()[:, None] / ts.double()[None, :]
  assert (cos.cpu().double() - torch.cos(exact)).abs().max() < 40000 * 2.0 ** -23


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("hq,hkv,dh,ps", [(4, 1, 16, 4), (6, 2, 48, 8), (3, 3, 256, 64), (8, 4, 112, 16)])
def test_rope_and_cache_write(table, dtype, hq, hkv, dh, ps):
  ops, ref = table[dtype], ReferenceOps(dtype)
  seqs = [(0, 9), (37, 1), (130, 21), (5, 2)]
  sc = make_scenario(seqs, num_kv_heads=hkv, head_dim=dh, window=None, page_size=ps, dtype=dtype,
                     device="cuda", ops=ops, seed=3)
  t = sc.ctx.num_tokens
  qkv = torch.randn(t, (hq + 2 * hkv) * dh).to(dtype).cuda()
  rot = ops.rotation_tables(sc.ctx.positions, torch.linspace(1, 900, dh // 2).cuda(), 1.0)
  st_ref = sc.storage.clone()
  q_ref = ref.rope_and_cache_write(qkv, rot, 0.37, hq, hkv, dh, st_ref, sc.block_table, sc.ctx)
  q = ops.rope_and_cache_write(qkv, rot, 0.37, hq, hkv, dh, sc.storage, sc.block_table, sc.ctx)
  ops.check_errors()
  close(q, q_ref, dtype, 3.0)
  # Written places agree; every other place of the cache is untouched (NaN stays NaN, values stay).
  torch.testing.assert_close(sc.storage.float().cpu(), st_ref.float().cpu(), equal_nan=True, **tol(dtype, 3.0))
  # No rotation, and a projection that holds q only (a layer that reads another layer's cache).
  q_only = torch.randn(t, hq * dh).to(dtype).cuda()
  close(ops.rope_and_cache_write(q_only, None, 1.0, hq, 0, dh, None, sc.block_table, sc.ctx).reshape(t, -1),
        q_only, dtype)


@pytest.mark.parametrize("hq,hkv,dh,ps,width", [(4, 1, 32, 4, 72), (6, 2, 96, 8, 200), (3, 3, 256, 64, 1000),
                                                 (8, 4, 64, 16, 520)])
@pytest.mark.parametrize("seqs", [[(0, 9), (37, 1), (130, 6)], [(5, 1)], [(63, 1), (64, 1), (200, 1), (7, 1), (0, 1)]],
                         ids=["mixed16", "one", "decode5"])
def test_project_rotate_store_fused(table, hq, hkv, dh, ps, width, seqs):
  """The one-kernel projection + rotation + cache write of small steps against the two-kernel path
  and the plain statement: queries, written cache rows, and nothing else touched."""
  dtype = torch.bfloat16
  ops, ref = table[dtype], ReferenceOps(dtype)
  sc = make_scenario(seqs, num_kv_heads=hkv, head_dim=dh, window=None, page_size=ps, dtype=dtype,
                     device="cuda", ops=ops, seed=5)
  t = sc.ctx.num_tokens
  assert t <= 16
  x = torch.randn(t, width).to(dtype).cuda()
  w = (torch.randn((hq + 2 * hkv) * dh, width) / width ** 0.5).to(dtype).cuda()
  rot = ops.rotation_tables(sc.ctx.positions, torch.linspace(1, 900, dh // 2).cuda(), 1.0)
  st_ref, st_two = sc.storage.clone(), sc.storage.clone()
  q_ref = ref.project_rotate_store(x, w, rot, 0.37, hq, hkv, dh, st_ref,
                                   sc.block_table, sc.ctx)
  before = ops.launches
  q = ops.project_rotate_store(x, w, rot, 0.37, hq, hkv, dh, sc.storage, sc.block_table, sc.ctx)
  assert ops.launches - before == 1  # one kernel
  ops.check_errors()
  ops.fused_qkv_rope = False
  try:
    q_two = ops.project_rotate_store(x, w, rot, 0.37, hq, hkv, dh, st_two, sc.block_table, sc.ctx)
  finally:
    ops.fused_qkv_rope = True
  close(q, q_ref, dtype, 3.0)
  close(q, q_two, dtype, 3.0)
  torch.testing.assert_close(sc.storage.float().cpu(), st_ref.float().cpu(), equal_nan=True, **tol(dtype, 3.0))
  torch.testing.assert_close(sc.storage.float().cpu(), st_two.float().cpu(), equal_nan=True, **tol(dtype, 3.0))
  # Without rotation and without a cache (a layer that reads another layer's cache).
  wq = w[:hq * dh]
  q_plain = ops.project_rotate_store(x, wq, None, 1.0, hq, 0, dh, None, sc.block_table, sc.ctx)
  close(q_plain.reshape(t, -1), ref.linear(x, wq), dtype, 3.0)


# ---- feed-forward pieces ---------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("act", [0, 1, 2])
def test_gated_activation(table, dtype, act):
  ops, ref = table[dtype], ReferenceOps(dtype)
  gu = (torch.randn(13, 2 * 330) * 3).to(dtype)
  close(ops.gated_activation(gu.cuda(), act), ref.gated_activation(gu, act), dtype, 3.0)


@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (5, 200, 72), (17, 1000, 96), (70, 130, 33), (130, 65, 300)])
def test_linear_float32_is_true_float32(table, m, n, k):
  ops = table[torch.float32]
  x, w = torch.randn(m, k), torch.randn(n, k)
  got = ops.linear(x.cuda(), w.cuda()).cpu()
  want = (x.double() @ w.double().t())
  # A reduced-precision matrix mode (TF32: 10-bit mantissa) would miss this by 100x.
  assert (got.double() - want).abs().max() < 1e-6 * k ** 0.5 * 8
  # The sum over K does not depend on what else is in the batch.
  alone = ops.linear(x[m // 2:m // 2 + 1].cuda(), w.cuda()).cpu()
  assert torch.equal(alone[0], got[m // 2])


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 17, 24, 32, 33, 47, 64, 65, 200])
@pytest.mark.parametrize("n,k", [(48, 64), (1000, 96), (2304, 2048), (100, 328), (130, 9216), (4096, 2304)])
def test_linear_bfloat16(table, m, n, k):
  ops, ref = table[torch.bfloat16], ReferenceOps(torch.bfloat16)
  x = torch.randn(m, k).to(torch.bfloat16)
  w = (torch.randn(n, k) / k ** 0.5).to(torch.bfloat16)
  close(ops.linear(x.cuda(), w.cuda()), ref.linear(x, w), torch.bfloat16)


@pytest.mark.parametrize("stages", [0, 4, 8])
@pytest.mark.parametrize("split", [0, 1, 2, 3, 6, 8])
@pytest.mark.parametrize("m,n,k", [(17, 128, 128), (33, 300, 1032), (64, 2304, 2048), (50, 257, 2304), (64, 129, 8),
                                   (100, 1000, 2304), (128, 2304, 9216)])
def test_serving_batch_product_with_k_split_over_a_cluster(table, stages, split, m, n, k):
  """The product for 17 to 128 tokens, with the sum over k in one block or split over the blocks of
  a cluster (their partial sums are added in rank order: the same result every time)."""
  ops, ref = table[torch.bfloat16], ReferenceOps(torch.bfloat16)
  x = torch.randn(m, k).to(torch.bfloat16).cuda()
  w = (torch.randn(n, k) / k ** 0.5).to(torch.bfloat16).cuda()
  ops.mid_split, ops.mid_stages = split, stages
  kept, ops.mid_rows = ops.mid_rows, dict.fromkeys(ops.mid_rows, 128)  # whatever the engine's own limit is
  try:
    before = ops.launches
    got = ops.linear(x, w)
    assert ops.launches == before + 1
    again = ops.linear(x, w)
  finally:
    ops.mid_split, ops.mid_stages, ops.mid_rows = 0, 0, kept
  ops.check_errors()
  close(got, ref.linear(x.cpu(), w.cpu()), torch.bfloat16)
  assert torch.equal(got, again)
  ops.mid_rows_kernel = False
  try:
    close(got, ops.linear(x, w), torch.bfloat16)  # the library product of the same shape
  finally:
    ops.mid_rows_kernel = True


@pytest.mark.parametrize("hq,hkv,dh,ps,width", [(3, 1, 128, 16, 200), (8, 4, 256, 64, 2304), (2, 2, 128, 8, 72)])
@pytest.mark.parametrize("seqs", [[(0, 17)], [(37, 1)] * 20 + [(130, 6), (5, 30)], [(200, 1)] * 64, [(0, 40), (90, 24)],
                                  [(3, 1)] * 90 + [(70, 38)]],
                         ids=["prompt17", "mixed56", "decode64", "two64", "mixed128"])
def test_project_rotate_store_fused_for_a_serving_batch(table, hq, hkv, dh, ps, width, seqs):
  """Steps of 17 to 128 tokens: projection, rotation, query scale and cache write in one kernel,
  against the two-kernel path and the plain statement."""
  dtype = torch.bfloat16
  ops, ref = table[dtype], ReferenceOps(dtype)
  kept, ops.mid_rows = ops.mid_rows, dict.fromkeys(ops.mid_rows, 128)
  try:
    _check_fused_serving_batch(ops, ref, dtype, hq, hkv, dh, ps, width, seqs)
  finally:
    ops.mid_rows = kept


def _check_fused_serving_batch(ops, ref, dtype, hq, hkv, dh, ps, width, seqs):
  sc = make_scenario(seqs, num_kv_heads=hkv, head_dim=dh, window=None, page_size=ps, dtype=dtype,
                     device="cuda", ops=ops, seed=6)
  t = sc.ctx.num_tokens
  assert 16 < t <= 128
  x = torch.randn(t, width).to(dtype).cuda()
  w = (torch.randn((hq + 2 * hkv) * dh, width) / width ** 0.5).to(dtype).cuda()
  rot = ops.rotation_tables(sc.ctx.positions, torch.linspace(1, 900, dh // 2).cuda(), 1.0)
  st_ref, st_two = sc.storage.clone(), sc.storage.clone()
  q_ref = ref.project_rotate_store(x, w, rot, 0.37, hq, hkv, dh, st_ref, sc.block_table, sc.ctx)
  before = ops.launches
  q = ops.project_rotate_store(x, w, rot, 0.37, hq, hkv, dh, sc.storage, sc.block_table, sc.ctx)
  assert ops.launches - before == 1  # one kernel
  ops.check_errors()
  ops.fused_qkv_rope = False
  try:
    q_two = ops.project_rotate_store(x, w, rot, 0.37, hq, hkv, dh, st_two, sc.block_table, sc.ctx)
  finally:
    ops.fused_qkv_rope = True
  close(q, q_ref, dtype, 3.0)
  close(q, q_two, dtype, 3.0)
  torch.testing.assert_close(sc.storage.float().cpu(), st_ref.float().cpu(), equal_nan=True, **tol(dtype, 3.0))
  torch.testing.assert_close(sc.storage.float().cpu(), st_two.float().cpu(), equal_nan=True, **tol(dtype, 3.0))
  wq = w[:hq * dh].contiguous()
  q_plain = ops.project_rotate_store(x, wq, None, 1.0, hq, 0, dh, None, sc.block_table, sc.ctx)
  close(q_plain.reshape(t, -1), ref.linear(x, wq), dtype, 3.0)


@pytest.mark.parametrize("m", [33, 64, 100, 700, 2048])
def test_library_product_is_called_directly(table, m):
  """Steps of more than 32 tokens: the library product, called by the package's own code with an
  algorithm kept per size class (one launch counted, no tensor-library call), gives what the
  tensor library's call gives, whichever row count of a class comes first."""
  ops, ref = table[torch.bfloat16], ReferenceOps(torch.bfloat16)
  n, k = 2304, 2048
  x = torch.randn(m, k).to(torch.bfloat16)
  w = (torch.randn(n, k) / k ** 0.5).to(torch.bfloat16)
  before = ops.launches
  got = ops.linear(x.cuda(), w.cuda())
  assert ops.launches == before + 1
  close(got, ref.linear(x, w), torch.bfloat16)
  ops.direct_library_products = False
  try:
    through_torch = ops.linear(x.cuda(), w.cuda())
    assert ops.launches == before + 1  # not one of the package's launches
  finally:
    ops.direct_library_products = True
  close(got, through_torch.cpu(), torch.bfloat16)


@pytest.mark.parametrize("m", [1, 8, 13, 17, 40, 64, 70, 128, 130])
@pytest.mark.parametrize("f,k,act", [(160, 96, 0), (1000, 64, 1), (9216 // 4, 2304, 0), (100, 2048, 2)])
def test_gated_linear(table, m, f, k, act):
  torch.manual_seed(1000 * m + f)
  for dtype, own_up_to in ((torch.float32, None), (torch.bfloat16, None), (torch.bfloat16, 128)):
    # (own_up_to = 128: the engine's own product with the activation in its epilogue for every
    # row count it takes, not only for those where it is faster than the library's)
    ops, ref = table[dtype], ReferenceOps(dtype)
    x = torch.randn(m, k).to(dtype)
    w = (torch.randn(2 * f, k) / k ** 0.5 * 2).to(dtype)
    kept = ops.mid_rows
    if own_up_to:
      ops.mid_rows = dict.fromkeys(kept, own_up_to)
    try:
      got, want = ops.gated_linear(x.cuda(), w.cuda(), act), ref.gated_linear(x, w, act)
    finally:
      ops.mid_rows = kept
    if dtype == torch.float32:
      close(got, want, dtype, 2.0)
    else:
      # Three bfloat16 roundings stand between the float32 sums and the result (gate, up, their
      # product), and two right implementations may land one unit in the last place (2^-8) apart
      # at each: 1.17 % at most, where the common bound for one rounding is 1 %.  (With unseeded
      # inputs this test met such an element about once in twenty runs.)
      torch.testing.assert_close(got.float().cpu(), want.float().cpu(), atol=2e-2, rtol=3.2 * 2.0 ** -8)


@pytest.mark.parametrize("pairs", [False, True])
@pytest.mark.parametrize("blocks", [0, 4])
@pytest.mark.parametrize("m,f,k,act", [(128, 128, 64, 0), (300, 384, 72, 1), (129, 256, 1032, 2), (1000, 1152, 2304, 0),
                                       (2048, 2304, 328, 0), (515, 640, 520, 1)])
def test_gated_product_for_many_tokens(table, pairs, blocks, m, f, k, act):
  """The tcgen05 product with the activation on its accumulators, by single blocks and by pairs of
  blocks: token counts that end inside a tile (or leave a pair's second block without a row), k
  that ends inside a stage, and so few blocks that each walks many tiles (both accumulators and
  every stage of the ring are used again and again)."""
  torch.manual_seed(m + f + k)
  ops, ref = table[torch.bfloat16], ReferenceOps(torch.bfloat16)
  x = torch.randn(m, k).to(torch.bfloat16)
  w = (torch.randn(2 * f, k) / k ** 0.5 * 2).to(torch.bfloat16)
  kept = ops.gated_tc_min_rows, ops.gated_tc_blocks, ops.gated_tc_pairs
  ops.gated_tc_min_rows, ops.gated_tc_blocks, ops.gated_tc_pairs = 1, blocks, pairs
  before = ops.launches
  try:
    got = ops.gated_linear(x.cuda(), w.cuda(), act)
  finally:
    ops.gated_tc_min_rows, ops.gated_tc_blocks, ops.gated_tc_pairs = kept
  ops.check_errors()
  assert ops.launches - before == 1, "the product and its activation are one kernel"
  # see test_gated_linear for the bound
  torch.testing.assert_close(got.float().cpu(), ref.gated_linear(x, w, act).float().cpu(), atol=2e-2,
                             rtol=3.2 * 2.0 ** -8)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("r,v,k,cap", [(1, 1000, 96, 10.0), (7, 256, 64, 30.0), (45, 1003, 72, 0.0), (3, 25600, 2304, 30.0),
                                       (40, 2048, 72, 30.0), (64, 25601, 2304, 30.0), (33, 130, 1000, 0.0), (100, 5000, 96, 30.0),
                                       (140, 1000, 96, 30.0)])
def test_lm_head(table, dtype, r, v, k, cap):
  ops, ref = table[dtype], ReferenceOps(dtype)
  x = (torch.randn(r, k) * 2).to(dtype)
  t = torch.randn(v, k).to(dtype)
  got = ops.lm_head(x.cuda(), t.cuda(), cap)
  assert got.dtype == torch.float32
  # The product is accumulated and capped in float32 in both dtypes.
  torch.testing.assert_close(got.cpu(), ref.lm_head(x, t, cap), atol=2e-4 * k ** 0.5, rtol=1e-4)
  if dtype == torch.bfloat16 and 32 < r <= 128:
    # the engine's own product with the soft cap in its epilogue, where the library's is the default
    kept, ops.mid_rows = ops.mid_rows, dict.fromkeys(ops.mid_rows, 128)
    try:
      own = ops.lm_head(x.cuda(), t.cuda(), cap)
    finally:
      ops.mid_rows = kept
    torch.testing.assert_close(own.cpu(), ref.lm_head(x, t, cap), atol=2e-4 * k ** 0.5, rtol=1e-4)


def test_weight_stored_in_32_bits_is_used_in_32_bits(table):
  ops = table[torch.bfloat16]
  x = torch.randn(4, 64).to(torch.bfloat16)
  w = torch.randn(32, 64)  # float32 although the engine runs in bfloat16
  got = ops.linear(x.cuda(), w.cuda())
  assert got.dtype == torch.bfloat16
  want = (x.float() @ w.t()).to(torch.bfloat16)
  assert torch.equal(got.cpu(), want) or (got.cpu().float() - want.float()).abs().max() <= 2 ** -7 * want.abs().max()


# ---- attention ---------------------------------------------------------------------
ATTN_CASES = [
    # hq, hkv, dh, page, window, cap
    (4, 1, 16, 4, 8, 50.0),
    (6, 2, 32, 8, 16, 20.0),
    (8, 4, 256, 64, None, 50.0),
    (8, 4, 256, 16, 100, 50.0),
    (3, 3, 48, 16, None, 0.0),
    (5, 1, 80, 32, 33, 30.0),
    (32, 16, 128, 64, 70, 50.0),
]
SEQS = [(0, 19), (250, 1), (64, 64), (3, 2), (129, 37), (511, 1)]


def run_attention(ops, q, sc, hq, hkv, dh, cap, window):
  return ops.paged_attention(q, sc.storage, sc.block_table, sc.ctx, num_heads=hq, num_kv_heads=hkv,
                             head_dim=dh, logit_softcap=cap, window=window)


@pytest.fixture
def general_bf16(table):
  """The bfloat16 table with the tensor-core attention switched off (the general kernel runs)."""
  ops = table[torch.bfloat16]
  ops.tensor_core_attention = False
  yield ops
  ops.tensor_core_attention = True


@pytest.mark.parametrize("hq,hkv,dh,ps,window,cap", ATTN_CASES)
def test_paged_attention_general_kernel_bfloat16(general_bf16, hq, hkv, dh, ps, window, cap):
  ops, ref = general_bf16, ReferenceOps(torch.bfloat16)
  sc = make_scenario(SEQS, num_kv_heads=hkv, head_dim=dh, window=window, page_size=ps, dtype=torch.bfloat16,
                     device="cuda", ops=ops, seed=5)
  q = (torch.randn(sc.ctx.num_tokens, hq, dh) * 1.5).to(torch.bfloat16).cuda()
  got = run_attention(ops, q, sc, hq, hkv, dh, cap, window)
  ops.check_errors()
  close(got, run_attention(ref, q, sc, hq, hkv, dh, cap, window), torch.bfloat16, 2.0)


@pytest.mark.parametrize("chunk,rows", [(64, 16), (128, 8), (0, 8), (256, 16), (64, 8)])
@pytest.mark.parametrize("hq,hkv,dh,ps,window,cap", ATTN_CASES)
def test_split_key_attention_chunks(table, chunk, rows, hq, hkv, dh, ps, window, cap):
  """Only short entries (the split-key kernels: up to 16 query rows per kv head, and the
  turned-round one for up to 8), long histories, several chunk lengths."""
  ops, ref = table[torch.bfloat16], ReferenceOps(torch.bfloat16)
  group = hq // hkv
  few = max(rows // group, 1)
  seqs = [(1000, 1), (0, 1), (63, 1), (64, few), (700, min(2, few)), (129, 1), (31, 1), (255, 1)]
  sc = make_scenario(seqs, num_kv_heads=hkv, head_dim=dh, window=window, page_size=ps, dtype=torch.bfloat16,
                     device="cuda", ops=ops, seed=6)
  q = (torch.randn(sc.ctx.num_tokens, hq, dh) * 1.5).to(torch.bfloat16).cuda()
  ops.decode_chunk = chunk
  want = run_attention(ref, q, sc, hq, hkv, dh, cap, window)
  try:
    # by row count (TMA with a producer warp where it can), without TMA, TMA without the producer warp, the 16-row kernel
    for variant in (0, 1, 2, 16):
      ops.decode_variant = variant
      got = run_attention(ops, q, sc, hq, hkv, dh, cap, window)
      ops.check_errors()
      assert torch.isfinite(got).all()
      close(got, want, torch.bfloat16, 2.0)
  finally:
    ops.decode_chunk = 0
    ops.decode_variant = 0


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("hq,hkv,dh,ps,window,cap", ATTN_CASES)
def test_paged_attention_random(table, dtype, hq, hkv, dh, ps, window, cap):
  ops, ref = table[dtype], ReferenceOps(dtype)
  sc = make_scenario(SEQS, num_kv_heads=hkv, head_dim=dh, window=window, page_size=ps, dtype=dtype,
                     device="cuda", ops=ops, seed=5)
  q = (torch.randn(sc.ctx.num_tokens, hq, dh) * 1.5).to(dtype).cuda()
  want = run_attention(ref, q, sc, hq, hkv, dh, cap, window)
  # Prefill kernels: tcgen05 where the shape allows; mma.sync with tiles of 64 rows (two key groups),
  # 64 rows with a single key group (written 65 here) and 128 rows.
  variants = [(False, 0)] if dtype == torch.float32 else [(True, 0), (True, 1), (False, 0), (False, 64), (False, 65), (False, 128)]
  for tc, rows in variants:
    ops.prefill_tcgen05 = tc
    ops.prefill_pairs = rows != 1  # (True, 1): tcgen05 by single blocks
    ops.prefill_rows = (64 if rows == 65 else rows) if rows >= max(hq // hkv, 2) else 0
    ops.prefill_single_key_group = rows == 65
    sc.ctx.memo.clear()
    try:
      got = run_attention(ops, q, sc, hq, hkv, dh, cap, window)
    finally:
      ops.prefill_tcgen05 = True
      ops.prefill_pairs = True
      ops.prefill_rows = 0
      ops.prefill_single_key_group = False
    ops.check_errors()
    assert torch.isfinite(got).all(), "a page the request does not hold was read"
    close(got, want, dtype, 2.0)


@pytest.mark.parametrize("hq,hkv,dh,ps,window,cap", [
    (8, 4, 256, 64, None, 0.0), (8, 4, 256, 64, 1000, 50.0), (4, 1, 64, 16, None, 30.0), (16, 8, 128, 64, 300, 0.0),
    (8, 1, 192, 32, None, 50.0)])
def test_tcgen05_prefill_long_walks(table, hq, hkv, dh, ps, window, cap):
  """Long portions through the tcgen05 prefill kernel: dozens of key tiles per block, so that its
  warps (loaders, two issuers, two softmax groups) hand over to each other many times, with
  scores spread so widely that the running maximum moves and O is rescaled again and again.
  Run a few times: a hand-over that can miss a phase shows as a timed-out wait or a wrong row."""
  dtype = torch.bfloat16
  ops, ref = table[dtype], ReferenceOps(dtype)
  seqs = [(700, 1900), (0, 130), (64, 1)]
  sc = make_scenario(seqs, num_kv_heads=hkv, head_dim=dh, window=window, page_size=ps, dtype=dtype,
                     device="cuda", ops=ops, seed=11)
  q = (torch.randn(sc.ctx.num_tokens, hq, dh) * 3.0).to(dtype).cuda()
  want = run_attention(ref, q, sc, hq, hkv, dh, cap, window)  # the plain statement
  for pairs in (True, False, True, False):  # by pairs of blocks where the shape allows, and by single blocks
    ops.prefill_pairs = pairs
    sc.ctx.memo.clear()
    try:
      got = run_attention(ops, q, sc, hq, hkv, dh, cap, window)
    finally:
      ops.prefill_pairs = True
    ops.check_errors()
    assert torch.isfinite(got).all()
    close(got, want, dtype, 2.0)


def test_a_cache_at_a_reused_address_gets_a_descriptor_of_its_own(table):
  """The decode kernels read the cache through a TMA descriptor that the kernel table keeps per
  storage.  A second, larger storage at the same address (another engine after the first one was
  freed) must not get the first one's descriptor: its rows would end too early and the keys of
  the higher pages would read as zeros."""
  dtype = torch.bfloat16
  ops, ref = table[dtype], ReferenceOps(dtype)
  hq, hkv, dh, ps = 4, 2, 64, 16
  arena = torch.zeros(8 * 1024 * 1024, dtype=dtype, device="cuda")
  for seqs in ([(40, 1)], [(900, 1), (500, 1), (30, 1)]):  # the second cache has many more pages
    sc = make_scenario(seqs, num_kv_heads=hkv, head_dim=dh, window=None, page_size=ps, dtype=dtype,
                       device="cuda", ops=ops, seed=4)
    at_same_address = arena[:sc.storage.numel()].view_as(sc.storage)
    at_same_address.copy_(sc.storage)
    assert at_same_address.data_ptr() == arena.data_ptr()
    q = torch.randn(sc.ctx.num_tokens, hq, dh).to(dtype).cuda()
    want = run_attention(ref, q, sc, hq, hkv, dh, 30.0, None)
    got = ops.paged_attention(q, at_same_address, sc.block_table, sc.ctx, num_heads=hq, num_kv_heads=hkv,
                              head_dim=dh, logit_softcap=30.0, window=None)
    ops.check_errors()
    close(got, want, dtype, 2.0)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("ps", [16, 64])
@pytest.mark.parametrize("window", [None, 96])
def test_paged_attention_one_key_stands_out(table, dtype, ps, window):
  """One key matches the query far better than the rest and carries a value of its own.
  Placed far back, at a page's edge and at the window's edge, it shows whether exactly
  the right keys are visible."""
  ops = table[dtype]
  hq, hkv, dh, cap = 4, 2, 64, 50.0
  hist = 700
  sc = make_scenario([(hist, 1), (hist, 3)], num_kv_heads=hkv, head_dim=dh, window=window, page_size=ps,
                     dtype=dtype, device="cuda", ops=ops, seed=9)
  g = sc.manager.groups[0]
  direction = torch.nn.functional.normalize(torch.randn(dh), dim=0)
  q = (direction * 9.0).expand(sc.ctx.num_tokens, hq, dh).contiguous().to(dtype).cuda()
  w = window if window is not None else 10 ** 9
  spots = [3, ps - 1, ps, hist - w, hist - w + 1, hist - w + 2, hist - 1, hist, hist + 1, hist + 2]
  for spot in spots:
    if spot < 0:
      continue
    backup = sc.storage.clone()
    for slot, q_start, q_len in sc.seqs:
      page = int(g.tables[slot, spot // ps])
      if page < 0 or spot >= q_start + q_len:
        continue  # given back (outside every window) or not yet there
      sc.storage[page, 0, :, spot % ps, :] = (direction * 9.0).to(dtype).cuda()
      sc.storage[page, 1, :, spot % ps, :] = 7.0
    got = run_attention(ops, q, sc, hq, hkv, dh, cap, window).float().cpu().reshape(sc.ctx.num_tokens, hq, dh)
    ops.check_errors()
    row = 0
    for slot, q_start, q_len in sc.seqs:
      for i in range(q_len):
        pos = q_start + i
        visible = spot <= pos and (window is None or pos - spot < window)
        mean = got[row].mean().item()
        if visible:
          assert mean > 6.5, (spot, pos, mean)  # e^(cap*tanh(81/50) - others) swamps ~700 ordinary keys
        else:
          assert abs(mean) < 1.0, (spot, pos, mean)
        row += 1
    sc.storage.copy_(backup)


@pytest.mark.parametrize("hq,hkv,dh,ps", [(4, 4, 128, 64), (8, 2, 256, 128), (16, 2, 128, 64), (8, 4, 256, 64), (4, 2, 64, 16)])
@pytest.mark.parametrize("window", [None, 200])
def test_prefill_attention_one_key_stands_out(table, hq, hkv, dh, ps, window):
  """Portions of prompts (the prefill kernels: by pairs of blocks, by single blocks, mma.sync),
  several groups and page sizes: one key matches every query far better than the rest and carries
  a value of its own.  Placed at a tile's, a page's and the window's edge, and where a pair's first
  block ends, it shows whether exactly the right keys are visible to exactly the right rows; the
  whole result is compared with the plain statement as well."""
  dtype = torch.bfloat16
  ops, ref = table[dtype], ReferenceOps(dtype)
  cap = 50.0
  seqs = [(300, 330), (0, 257), (1000, 70)]
  sc = make_scenario(seqs, num_kv_heads=hkv, head_dim=dh, window=window, page_size=ps, dtype=dtype,
                     device="cuda", ops=ops, seed=13)
  g = sc.manager.groups[0]
  direction = torch.nn.functional.normalize(torch.randn(dh), dim=0)
  q = (direction * 9.0).expand(sc.ctx.num_tokens, hq, dh).contiguous().to(dtype).cuda()
  tokens_per_block = 128 // (hq // hkv)
  for variant in ("pairs", "single", "mma"):
    ops.prefill_pairs, ops.prefill_tcgen05 = variant == "pairs", variant != "mma"
    try:
      for spot in (0, 63, 64, 127, 128, 299, 300, 300 + tokens_per_block - 1, 300 + tokens_per_block, 430, 629, 1001):
        backup = sc.storage.clone()
        for slot, q_start, q_len in sc.seqs:
          page = int(g.tables[slot, spot // ps]) if spot < q_start + q_len else -1
          if page < 0:
            continue  # given back (outside every window) or not yet there
          sc.storage[page, 0, :, spot % ps, :] = (direction * 9.0).to(dtype).cuda()
          sc.storage[page, 1, :, spot % ps, :] = 7.0
        sc.ctx.memo.clear()
        got = run_attention(ops, q, sc, hq, hkv, dh, cap, window)
        ops.check_errors()
        close(got, run_attention(ref, q, sc, hq, hkv, dh, cap, window), dtype, 2.0)
        got = got.float().cpu().reshape(sc.ctx.num_tokens, hq, dh)
        row = 0
        for slot, q_start, q_len in sc.seqs:
          for i in range(q_len):
            pos = q_start + i
            visible = spot <= pos and (window is None or pos - spot < window)
            mean = got[row].mean().item()
            if visible:
              assert mean > 6.5, (variant, spot, pos, mean)
            else:
              assert abs(mean) < 1.0, (variant, spot, pos, mean)
            row += 1
        sc.storage.copy_(backup)
    finally:
      ops.prefill_pairs = ops.prefill_tcgen05 = True


# ---- sampling ---------------------------------------------------------------------
def test_sample_greedy_and_ties(table):
  ops = table[torch.float32]
  logits = torch.randn(5, 1003)
  logits[2, 17] = logits[2, 900] = 9.0  # lowest index wins a tie
  got = ops.sample(logits.cuda(), [0.0] * 5, [-1] * 5, [1.0] * 5, [0] * 5, [3] * 5).cpu()
  want = torch.tensor([int(torch.argmax(r)) for r in logits])
  want[2] = 17
  assert torch.equal(got.long(), want)
  got = ops.sample(logits.cuda(), [0.7] * 5, [1] * 5, [1.0] * 5, [0] * 5, [3] * 5).cpu()
  assert torch.equal(got.long(), want)  # top_k == 1 is greedy


@pytest.mark.parametrize("vocab", [256, 1003, 25601])
def test_sample_matches_plain_statement(table, vocab):
  ops = table[torch.float32]
  rng = np.random.default_rng(vocab)
  rows = 24
  logits = torch.from_numpy(rng.normal(size=(rows, vocab)).astype(np.float32) * 3)
  temperature = [0.8, 1.0, 0.3, 1.7] * (rows // 4)
  top_k = [-1, 5, -1, 40, 7, -1] * (rows // 6)
  top_p = [1.0, 1.0, 0.9, 0.5, 0.95, 0.2] * (rows // 6)
  seed = [int(rng.integers(0, 2 ** 63)) for _ in range(rows)]
  position = [int(rng.integers(1, 8192)) for _ in range(rows)]
  got = ops.sample(logits.cuda(), temperature, top_k, top_p, seed, position).cpu().tolist()
  want = [plain.sample_token(logits[i].numpy(), temperature[i], top_k[i], top_p[i], seed[i], position[i])
          for i in range(rows)]
  assert got == want
  # the same draw with the tokens' log-probabilities (simply/utils/sampling_lib.py:540-601)
  temperature[3], top_k[6] = 0.0, 1  # two greedy rows: log-probability 0
  tokens, logprobs = ops.sample(logits.cuda(), temperature, top_k, top_p, seed, position, logprobs=True)
  want_lp = [plain.token_logprob(logits[i].numpy(), int(tokens[i]), temperature[i], top_k[i], top_p[i])
             for i in range(rows)]
  np.testing.assert_allclose(logprobs.cpu().numpy(), want_lp, atol=1e-4)
  assert logprobs[3] == 0 and logprobs[6] == 0 and (logprobs <= 0).all()


def test_sample_is_distributed_as_softmax(table):
  ops = table[torch.float32]
  logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5]]).repeat(4000, 1)
  got = ops.sample(logits.cuda(), [1.0] * 4000, [-1] * 4000, [1.0] * 4000, list(range(4000)), [5] * 4000)
  freq = torch.bincount(got.cpu().long(), minlength=5).float() / 4000
  want = torch.softmax(logits[0], 0)
  assert (freq - want).abs().max() < 0.03
