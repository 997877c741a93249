"""How close the engine's logits must be to the plain model's.

The bounds are fixed multiples of the rounding noise that is inherent to the
arithmetic, measured once with the plain PyTorch kernel statements on a CPU:
in float32 the engine differs from a float64 evaluation by about 1e-6 of the
largest logit (sums in another order, a few ulp in tanh/exp/sin/cos); with
bfloat16 activations (8 mantissa bits, rounded after every part) by about 0.9 %
of the largest logit at worst and 0.12 % on average.  The bounds are about
thirty times the former and three to four times the latter.
"""

import numpy as np

F32_MAX = 3e-5   # max |diff| / max |logit|
BF16_MAX = 3e-2
BF16_MEAN = 5e-3


def assert_logits_close(got, want, dtype, what=""):
  got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
  assert got.shape == want.shape, (what, got.shape, want.shape)
  assert np.isfinite(got).all(), f"{what}: logits are not finite"
  scale = np.abs(want).max()
  err = np.abs(got - want)
  if dtype == "float32":
    assert err.max() <= F32_MAX * scale, f"{what}: max diff {err.max():.3e} of scale {scale:.3e}"
  else:
    assert err.max() <= BF16_MAX * scale, f"{what}: max diff {err.max():.3e} of scale {scale:.3e}"
    assert err.mean() <= BF16_MEAN * scale, f"{what}: mean diff {err.mean():.3e} of scale {scale:.3e}"


def first_bad_position(got_rows, want, dtype):
  """Index of the first position whose logits are out of bounds (None if all are fine)."""
  bound = F32_MAX if dtype == "float32" else BF16_MAX
  scale = np.abs(want).max()
  for pos in sorted(got_rows):
    if not np.isfinite(got_rows[pos]).all() or np.abs(got_rows[pos] - want[pos]).max() > bound * scale:
      return pos
  return None
