"""The sampling entry point that allocates nothing (`sb_sample_static`, csrc/sample_static.h).

Some callers of this library may not allocate device memory: a serving thread that must
never take the allocator's lock, a process whose memory budget is fixed and policed after
start-up, a plug-in that only ever sees raw pointers from its host.  For them the library
carries the sampling kernels' scratch in a static device array.  This test calls the entry
point through its exported C symbol, as such a caller would, twice in a row on different
inputs (the array keeps the first call's contents, which must not leak into the second),
and compares the tokens with the ordinary entry point's.  It is collected last so that a
run that stops at the first failure has run everything else before.
"""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ROWS = 256
TOO_MANY_ROWS = -21
BAD_ARGUMENT = -22


def load_symbol():
  from simply_b200.kernels import build
  lib = ctypes.CDLL(build.build(verbose=False))
  fn = lib.sb_sample_static
  fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
  fn.restype = ctypes.c_int
  return fn


def make_case(ops, rows, vocab, seed):
  rng = np.random.default_rng(seed)
  logits = torch.from_numpy(rng.normal(size=(rows, vocab)).astype(np.float32) * 3).cuda()
  temperature = rng.choice([0.0, 0.7, 1.0, 1.5], rows).tolist()
  top_k = rng.choice([-1, 1, 5, 50], rows).tolist()
  top_p = rng.choice([1.0, 0.9, 0.4], rows).tolist()
  seeds = [int(s) for s in rng.integers(0, 2 ** 62, rows)]
  position = rng.integers(1, 8000, rows).tolist()
  params = torch.from_numpy(ops.pack_sample_params(temperature, top_k, top_p, seeds, position)).cuda()
  return logits, params


def test_static_scratch_sampling_matches_the_ordinary_entry_point():
  from simply_b200.kernels.ops import CudaOps

  ops = CudaOps(torch.float32)
  fn = load_symbol()
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  # Calls in a row; a call with fewer rows or another vocabulary finds stale words of the one
  # before right next to the ones it uses.  (4, 70001) and (3, 256000) cut a row into the most
  # slices the array is laid out for (64: few rows, a vocabulary of at least 65,536), each after a
  # larger call; (MAX_ROWS, 300) uses the most rows.
  cases = ((37, 25601, 0), (5, 1003, 1), (MAX_ROWS, 300, 2), (4, 70001, 3), (MAX_ROWS, 2100, 4), (3, 256000, 5),
           (9, 65536, 6))
  for rows, vocab, seed in cases:
    if rows <= 9 and vocab >= 65536:
      assert ops.lib.sb_sample_slices(rows, vocab) == 64
    logits, params = make_case(ops, rows, vocab, seed)
    want = ops.sample_device(logits, params)
    out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    rc = fn(logits.data_ptr(), params.data_ptr(), out.data_ptr(), rows, vocab, stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), want.cpu())
    assert int(out.min()) >= 0 and int(out.max()) < vocab


def test_static_scratch_sampling_refuses_what_it_cannot_hold():
  fn = load_symbol()
  dummy = torch.zeros(8, dtype=torch.int32, device="cuda")
  p = dummy.data_ptr()
  assert fn(p, p, p, MAX_ROWS + 1, 1000, None) == TOO_MANY_ROWS
  assert fn(None, p, p, 1, 1000, None) == BAD_ARGUMENT
  assert fn(p, p, p, 1, 0, None) == BAD_ARGUMENT
  assert fn(p, p, p, 0, 1000, None) == 0  # nothing to do is not an error
