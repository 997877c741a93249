"""Literal cases and formulas of the reference's own tests, restated against the plain model.

google-deepmind/simply cannot be imported without JAX, so its outputs cannot anchor the plain
model.  Its tests, read as text, still pin several conventions with literal numbers or with
formulas written out in NumPy.  Each case below names the test it restates:

* simply/model_lib_test.py:483-541: window masks for window_size 1 and 2 (a query sees
  window_size older keys plus itself), and a decode-time mask.
* simply/utils/rpa_shard_window_repro_test.py:86-111: float64 windowed grouped attention.
* simply/utils/testdata/ckpt_gemma2_format.json and ckpt_expected_format.json
  (simply/utils/checkpoint_lib_test.py:87-106): tensor layouts of the Gemma tree and of the
  reference's own tree; simply/utils/checkpoint_lib.py:423-496 maps model-folder names to that
  tree.
* simply/utils/sampling_lib_test.py:99-200: properties of the top-k and top-p masks.
* simply/utils/position_encoding_test.py:23-78: properties of the rotary encoding.
"""

import numpy as np
import pytest

from tests.plain import gemma2_plain as plain


# ---- masks -------------------------------------------------------------------------------


def _mask_of_segments(segment_ids, segment_positions, window_size):
  """The plain model's mask for packed segments: one sequence per segment id; the reference's
  window_size excludes the query, the plain model's window includes it."""
  ids, pos = np.asarray(segment_ids), np.asarray(segment_positions)
  n = len(ids)
  mask = np.zeros((n, n), bool)
  for s in np.unique(ids):
    where = np.nonzero(ids == s)[0]
    window = None if window_size is None else window_size + 1
    mask[np.ix_(where, where)] = plain.attention_mask(pos[where], pos[where], window)
  return mask


def test_window_masks_of_the_reference_tests():
  # simply/model_lib_test.py:483-520, window_size=1
  want0 = [[1, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0], [0, 1, 1, 0, 0, 0],
           [0, 0, 1, 1, 0, 0], [0, 0, 0, 0, 1, 0], [0, 0, 0, 0, 1, 1]]
  want1 = [[1, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0], [0, 1, 1, 0, 0, 0],
           [0, 0, 0, 1, 0, 0], [0, 0, 0, 1, 1, 0], [0, 0, 0, 0, 1, 1]]
  got0 = _mask_of_segments([1, 1, 1, 1, 2, 2], [0, 1, 2, 3, 0, 1], 1)
  got1 = _mask_of_segments([1, 1, 1, 2, 2, 2], [0, 1, 2, 0, 1, 2], 1)
  np.testing.assert_array_equal(got0, np.array(want0, bool))
  np.testing.assert_array_equal(got1, np.array(want1, bool))
  # simply/model_lib_test.py:522-541, window_size=2
  want = [[1, 0, 0, 0], [1, 1, 0, 0], [1, 1, 1, 0], [0, 1, 1, 1]]
  np.testing.assert_array_equal(_mask_of_segments([1] * 4, np.arange(4), 2), np.array(want, bool))
  # window_size=3 (the chunked-attention test's, :556): the fifth query sees keys 1..4
  m = _mask_of_segments([1] * 9, np.arange(9), 3)
  assert m[4].tolist() == [False, True, True, True, True, False, False, False, False]
  assert m.sum(axis=1).tolist() == [1, 2, 3, 4, 4, 4, 4, 4, 4]


def test_decode_mask_of_the_reference_tests():
  # simply/model_lib_test.py:543-554: a query at position 7 over keys at 3..7 sees them all
  m = plain.attention_mask([7], [3, 4, 5, 6, 7], None)
  assert m.tolist() == [[True] * 5]


# ---- attention ------------------------------------------------------------------------------


def _windowed_attention_float64(q, k, v, window_size):
  """The formula of simply/utils/rpa_shard_window_repro_test.py:86-111, written out again:
  queries are the last q_len positions of kv_len; mask keeps q_pos >= kv_pos and
  q_pos < kv_pos + window_size + 1; softmax over the kept scores; no soft cap, no scale."""
  q_len, hq, d = q.shape
  kv_len, hkv, _ = k.shape
  g = hq // hkv
  out = np.zeros((q_len, hq, d))
  for t in range(q_len):
    qp = kv_len - q_len + t
    lo = 0 if window_size is None else max(qp - window_size, 0)
    for n in range(hq):
      m = n // g
      s = k[lo:qp + 1, m].astype(np.float64) @ q[t, n].astype(np.float64)
      p = np.exp(s - s.max())
      out[t, n] = (p / p.sum()) @ v[lo:qp + 1, m].astype(np.float64)
  return out


@pytest.mark.parametrize("window_size", [None, 1, 5, 12, 64])
def test_grouped_attention_equals_the_reference_tests_formula(window_size):
  rng = np.random.default_rng(11)
  q_len, kv_len, hq, hkv, d = 7, 40, 6, 2, 8
  q = rng.normal(size=(q_len, hq, d))
  k = rng.normal(size=(kv_len, hkv, d))
  v = rng.normal(size=(kv_len, hkv, d))
  want = _windowed_attention_float64(q, k, v, window_size)
  window = None if window_size is None else window_size + 1
  got = plain.grouped_attention(q, k, v, np.arange(kv_len - q_len, kv_len), np.arange(kv_len), 0.0, window)
  np.testing.assert_allclose(got, want, atol=1e-12)


# ---- tensor layouts -----------------------------------------------------------------------------

# Layer 0 of the two fixtures (width 4, 2 heads of size 4, feed-forward 8).
_GEMMA_ATTN_VEC = np.array(  # attn_vec_einsum/w [N, H, D]
    [[[0, 8, 16, 24], [1, 9, 17, 25], [2, 10, 18, 26], [3, 11, 19, 27]],
     [[4, 12, 20, 28], [5, 13, 21, 29], [6, 14, 22, 30], [7, 15, 23, 31]]])
_GEMMA_QKV_Q = np.array(  # qkv_einsum/w[0] [N, D, H]
    [[[36, 37, 38, 39], [44, 45, 46, 47], [52, 53, 54, 55], [60, 61, 62, 63]],
     [[40, 41, 42, 43], [48, 49, 50, 51], [56, 57, 58, 59], [64, 65, 66, 67]]])
_GEMMA_GATING_FIRST_ROW = (180, 140)  # gating_einsum/w[0][0][0], w[1][0][0]
_SIMPLY_O = np.arange(0, 32).reshape(4, 2, 4)  # o_proj/w [D, N, H]
_SIMPLY_Q = np.arange(36, 68).reshape(4, 2, 4)  # q_proj/w [D, N, H]
_SIMPLY_UP_FIRST, _SIMPLY_GATE_FIRST = 140, 180  # ffn_0/w[0][0], ffn_0_gate/w[0][0]


def test_gemma_tree_and_reference_tree_hold_the_same_numbers():
  """What simply/utils/checkpoint_lib.py:256-335 does to the Gemma tree, on the fixtures' own
  numbers: 'nhd->dnh' for the output projection, 'ndh->dnh' for q; gating_einsum[0] is the
  gate (ffn_0_gate) and [1] the up projection (ffn_0)."""
  np.testing.assert_array_equal(np.einsum("nhd->dnh", _GEMMA_ATTN_VEC), _SIMPLY_O)
  np.testing.assert_array_equal(np.einsum("ndh->dnh", _GEMMA_QKV_Q), _SIMPLY_Q)
  assert _GEMMA_GATING_FIRST_ROW == (_SIMPLY_GATE_FIRST, _SIMPLY_UP_FIRST)


def test_model_folder_layouts_mean_what_the_reference_computes():
  """The model folder's [out, in] matrices, used the way the plain model uses them, give what the
  reference's einsums give on its own [D, N, H] tensors (simply/model_lib.py:2037-2072, :2362)
  when the two are related as simply/utils/checkpoint_lib.py:434-449 relates them:
  q_proj.weight.reshape(N, H, D) -> 'nhd->dnh'; o_proj.weight.reshape(D, N, H)."""
  d_model, n, h = _SIMPLY_Q.shape
  rng = np.random.default_rng(5)
  x = rng.normal(size=(3, d_model))
  w_q = _SIMPLY_Q.astype(np.float64)
  folder_q = np.einsum("dnh->nhd", w_q).reshape(n * h, d_model)  # inverse of 'nhd->dnh'
  want_q = np.einsum("ihd,ti->thd", w_q, x)  # 'ihd,...i->...hd'
  np.testing.assert_allclose((x @ folder_q.T).reshape(3, n, h), want_q)
  w_o = _SIMPLY_O.astype(np.float64)
  folder_o = w_o.reshape(d_model, n * h)  # inverse of _split_head(axis=1)
  heads = rng.normal(size=(3, n, h))
  want_o = np.einsum("ihd,thd->ti", w_o, heads)  # 'ihd,...hd->...i'
  np.testing.assert_allclose(heads.reshape(3, n * h) @ folder_o.T, want_o)
  # up/gate/down are plain transposes (:449-457): y @ w.T with w [out, in] is y @ ffn_w with [in, out]
  w_up = rng.normal(size=(8, d_model))
  np.testing.assert_allclose(x @ w_up.T, x @ np.transpose(w_up).copy())


def test_gate_is_the_activated_projection():
  """simply/model_lib.py:722-726: the activation acts on ffn_0_gate, not on ffn_0."""
  rng = np.random.default_rng(6)
  y = rng.normal(size=(2, 4))
  w_gate, w_up, w_down = rng.normal(size=(8, 4)), rng.normal(size=(8, 4)), rng.normal(size=(4, 8))
  want = (plain.gelu_tanh(y @ w_gate.T) * (y @ w_up.T)) @ w_down.T
  np.testing.assert_allclose(plain.gated_feed_forward(y, w_gate, w_up, w_down), want)
  swapped = plain.gated_feed_forward(y, w_up, w_gate, w_down)
  assert np.abs(swapped - want).max() > 1e-3


# ---- sampling masks ----------------------------------------------------------------------------


@pytest.mark.parametrize("top_k", [1, 5, 10, 12])
def test_top_k_mask_properties(top_k):
  # simply/utils/sampling_lib_test.py:99-114, :182-192
  rng = np.random.default_rng(0)
  for logits in rng.normal(size=(20, 10)).astype(np.float32):
    mask = plain.top_k_mask(logits, top_k)
    assert mask.sum() == min(top_k, 10)
    if (~mask).any():
      assert logits[~mask].max() < logits[mask].min()


@pytest.mark.parametrize("top_p", [0.2, 0.5, 0.8, 1.0])
def test_top_p_mask_properties(top_p):
  # simply/utils/sampling_lib_test.py:116-136
  rng = np.random.default_rng(0)
  for logits in rng.normal(size=(20, 10)).astype(np.float32):
    probs = np.exp(logits - logits.max())
    probs /= probs.sum()
    mask = plain.top_p_mask(logits, top_p)
    assert probs[mask].sum() + 1e-6 > top_p
    if (~mask).any():
      assert logits[~mask].max() < logits[mask].min()


def test_sampled_tokens_lie_inside_both_masks():
  # simply/utils/sampling_lib_test.py:138-152, :194-221
  rng = np.random.default_rng(1)
  for i, logits in enumerate(rng.normal(size=(15, 10)).astype(np.float32)):
    for top_k, top_p in ((3, 0.5), (2, 0.5), (5, 0.95), (10, 0.5)):
      tok = plain.sample_token(logits, 1.0, top_k, top_p, seed=i, position=3)
      assert plain.top_k_mask(logits, top_k)[tok]
      inner = np.where(plain.top_k_mask(logits, top_k), logits, -np.inf).astype(np.float32)
      assert plain.top_p_mask(inner, top_p)[tok]
  logits = rng.normal(size=50).astype(np.float32)
  assert plain.sample_token(logits, 0.0, -1, 1.0, 0, 0) == int(logits.argmax())  # :257-262
  assert plain.sample_token(logits, 1.0, 1, 1.0, 0, 0) == int(logits.argmax())  # :264-269
  a = [plain.sample_token(logits, 1.0, -1, 1.0, 9, p) for p in range(8)]
  assert a == [plain.sample_token(logits, 1.0, -1, 1.0, 9, p) for p in range(8)]  # :276, same seed


# ---- rotary encoding -------------------------------------------------------------------------


def test_rotary_properties_of_the_reference_tests():
  # simply/utils/position_encoding_test.py:23-78
  x = np.ones((4, 1, 64), np.float32)
  r = plain.rope(x, np.arange(4), 10_000.0)
  assert r.shape == x.shape and r.dtype == x.dtype
  assert not np.allclose(r[0], r[1])
  assert not np.allclose(plain.rope(x, [0, 1, 2, 3], 10_000.0), plain.rope(x, [0, 1, 0, 1], 10_000.0))
  np.testing.assert_array_equal(plain.rope(x, [0, 1, 0, 1], 10_000.0)[:2], plain.rope(x, [0, 1, 0, 1], 10_000.0)[2:])
  assert not np.allclose(r, plain.rope(x, np.arange(4), 1_000_000.0))
  assert not np.allclose(r, plain.rope(x, np.arange(4), 10_000.0, scale_factor=8.0))
  # position / scale_factor: eight times the position at scale 8 is the same angle
  np.testing.assert_allclose(plain.rope(x, [8], 10_000.0, scale_factor=8.0), plain.rope(x, [1], 10_000.0), rtol=1e-6)
