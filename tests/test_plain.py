"""The plain NumPy model checks itself: properties that follow from the formulas."""

import numpy as np
import pytest

from tests.plain import gemma2_plain as plain
from tests.tiny_models import write_tiny


def test_rope_keeps_norms_and_relative_angles():
  rng = np.random.default_rng(0)
  x = rng.normal(size=(9, 3, 32)).astype(np.float64)
  pos = np.array([0, 1, 2, 5, 9, 100, 1000, 4095, 8191])
  y = plain.rope(x, pos, 10000.0)
  np.testing.assert_allclose(np.linalg.norm(y, axis=-1), np.linalg.norm(x, axis=-1), rtol=1e-12)
  np.testing.assert_allclose(y[0], x[0])  # position 0 rotates nothing
  # q.k depends on the distance only
  q, k = rng.normal(size=(1, 1, 32)), rng.normal(size=(1, 1, 32))
  a = (plain.rope(q, [7], 10000.0) * plain.rope(k, [3], 10000.0)).sum()
  b = (plain.rope(q, [104], 10000.0) * plain.rope(k, [100], 10000.0)).sum()
  assert abs(a - b) < 1e-9
  # halves rotate together: dimension j pairs with j + half
  e = np.zeros((1, 1, 8)); e[0, 0, 1] = 1.0
  r = plain.rope(e, [1], 10000.0)[0, 0]
  assert np.count_nonzero(np.abs(r) > 1e-12) == 2 and r[1] != 0 and r[5] != 0


def test_window_lets_a_query_see_exactly_w_keys():
  pos = np.arange(20)
  m = plain.attention_mask(pos, pos, 8)
  assert m.sum(axis=1).tolist() == [min(i + 1, 8) for i in range(20)]
  assert m[10, 10] and m[10, 3] and not m[10, 2] and not m[10, 11]
  assert plain.attention_mask(pos, pos, None).sum() == 20 * 21 // 2


def test_soft_cap_and_gelu():
  x = np.array([-1e4, -3.0, 0.0, 3.0, 1e4])
  y = plain.soft_cap(x, 30.0)
  assert np.all(np.abs(y) <= 30.0) and y[2] == 0 and abs(y[3] - 30 * np.tanh(0.1)) < 1e-12
  assert plain.soft_cap(x, 0.0) is x
  g = plain.gelu_tanh(np.array([-10.0, 0.0, 10.0]))
  np.testing.assert_allclose(g, [0.0, 0.0, 10.0], atol=1e-6)


def test_rms_norm_has_unit_rms_before_scale():
  rng = np.random.default_rng(1)
  x = rng.normal(size=(4, 96)) * 7
  y = plain.rms_norm(x, np.zeros(96), 1e-6)
  np.testing.assert_allclose(np.sqrt((y ** 2).mean(-1)), 1.0, rtol=1e-6)
  np.testing.assert_allclose(plain.rms_norm(x, np.ones(96), 1e-6), 2 * y)
  np.testing.assert_allclose(plain.rms_norm(x, np.ones(96), 1e-6, plus_one=False), y)


def test_attention_rows_are_convex_combinations():
  rng = np.random.default_rng(2)
  t, hq, hkv, dh = 12, 6, 2, 8
  q, k = rng.normal(size=(t, hq, dh)), rng.normal(size=(t, hkv, dh))
  v = np.ones((t, hkv, dh)) * np.arange(t)[:, None, None]
  o = plain.grouped_attention(q, k, v, np.arange(t), np.arange(t), 50.0, 4)
  # values are the key's position: the output lies inside the window's range of positions
  for i in range(t):
    assert o[i].min() >= max(i - 3, 0) - 1e-9 and o[i].max() <= i + 1e-9
  # query heads 0..2 read kv head 0, heads 3..5 read kv head 1
  v2 = v.copy(); v2[:, 1] += 100
  o2 = plain.grouped_attention(q, k, v2, np.arange(t), np.arange(t), 50.0, 4)
  np.testing.assert_allclose(o2[:, :3], o[:, :3]); np.testing.assert_allclose(o2[:, 3:], o[:, 3:] + 100)


@pytest.mark.parametrize("which", ["a", "b"])
def test_float32_and_float64_agree_and_prefix_is_causal(tmp_path, which):
  folder = write_tiny(which, tmp_path, "bfloat16")
  m32, m64 = plain.PlainGemma2(folder, np.float32), plain.PlainGemma2(folder, np.float64)
  toks = np.random.default_rng(3).integers(0, m32.cfg["vocab_size"], 50).tolist()
  a, b = m32.forward(toks), m64.forward(toks)
  assert np.abs(a - b).max() < 1e-5 * np.abs(b).max()
  np.testing.assert_allclose(m64.forward(toks[:20]), b[:20], atol=1e-12)  # later tokens change nothing
  assert np.abs(b).max() <= m32.cfg["final_logit_softcapping"]


def test_philox_known_answers():
  # Random123 known-answer vectors for philox4x32-10.
  out = plain.philox4x32([[0], [0], [0], [0]], (0, 0))
  assert [int(x[0]) for x in out] == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
  f = 0xFFFFFFFF
  out = plain.philox4x32([[f], [f], [f], [f]], (f, f))
  assert [int(x[0]) for x in out] == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
  out = plain.philox4x32([[0x243f6a88], [0x85a308d3], [0x13198a2e], [0x03707344]], (0xa4093822, 0x299f31d0))
  assert [int(x[0]) for x in out] == [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]


def test_sampling_masks():
  logits = np.log(np.array([0.5, 0.25, 0.125, 0.0625, 0.0625], np.float32))
  assert plain.top_k_mask(logits, 2).tolist() == [True, True, False, False, False]
  assert plain.top_p_mask(logits, 0.7).tolist() == [True, True, False, False, False]
  assert plain.top_p_mask(logits, 0.5).tolist() == [True, False, False, False, False]
  assert plain.top_p_mask(logits, 1.0).all()
  assert plain.sample_token(logits, 0.0, -1, 1.0, 0, 0) == 0
  assert plain.sample_token(logits, 1.0, 1, 1.0, 0, 0) == 0
  draws = [plain.sample_token(logits, 1.0, -1, 1.0, s, 4) for s in range(3000)]
  freq = np.bincount(draws, minlength=5) / 3000
  assert np.abs(freq - np.exp(logits)).max() < 0.03
  assert set(plain.sample_token(logits, 1.0, 2, 1.0, s, 4) for s in range(200)) == {0, 1}


def test_plain_model_matches_its_committed_outputs():
  """tests/golden/plain_tiny.npz was written by tests/golden/make_golden.py (float64)."""
  import os
  from tests.golden.make_golden import compute
  path = os.path.join(os.path.dirname(__file__), "golden", "plain_tiny.npz")
  golden = np.load(path)
  for which, logits in compute().items():
    np.testing.assert_allclose(logits, golden[which], atol=1e-6)
