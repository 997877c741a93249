"""Plain, slow NumPy implementation of the Gemma 2 dense decoder: the tests' yardstick.

It rests on the reference's formulas only.  google-deepmind/simply cannot be
imported on a machine without JAX (simply/model_lib.py:28-51 imports jax, the
Pallas TPU ops, orbax and etils), so no output of the reference's own code
anchors this file; every function cites the lines it restates instead.

Whole sequences, no cache, one function per part.  It shares no code with the
engine: it reads config.json and the safetensors file with the `safetensors`
package and works on NumPy arrays in one dtype (`float32` as the reference's
tests do, simply/model_lib_test.py:60, or `float64`).
"""

from __future__ import annotations

import json
import os

import numpy as np

# ----------------------------------------------------------------------------
# Parts
# ----------------------------------------------------------------------------


def embed(tokens, table, dtype=np.float32):
  """simply/utils/module.py:450-481: rows of the table times sqrt(width).

  (`embedding_scale_by_sqrt_dim` = `embedding_lookup_scale` = 1.0, simply/config_lib.py:295.)
  """
  table = np.asarray(table, dtype)
  width = table.shape[1]
  return table[np.asarray(tokens, np.int64)] * dtype(np.sqrt(dtype(width)))


def rms_norm(x, scale, eps, plus_one=True):
  """simply/model_lib.py:154-178 with use_bias=False: no mean subtraction,
  x * rsqrt(mean(x^2) + eps) * (1 + scale)."""
  dtype = x.dtype
  var = np.mean(np.square(x), axis=-1, keepdims=True, dtype=dtype)
  y = x * (dtype.type(1.0) / np.sqrt(var + dtype.type(eps)))
  w = np.asarray(scale, dtype)
  return y * (w + dtype.type(1.0) if plus_one else w)


def rope(x, positions, theta, scale_factor=1.0):
  """simply/utils/position_encoding.py:83-110: x is [T, heads, head_dim]; the halves
  (first, second) rotate together; timescale_j = theta ** (2j / head_dim)."""
  dtype = x.dtype
  dh = x.shape[-1]
  half = dh // 2
  fraction = (2 * np.arange(half) / dh).astype(dtype)
  timescale = np.power(dtype.type(theta), fraction).astype(dtype)
  pos = np.asarray(positions, dtype)[:, None, None]
  angle = pos / timescale[None, None, :] / dtype.type(scale_factor)
  sin, cos = np.sin(angle), np.cos(angle)
  first, second = x[..., :half], x[..., half:]
  return np.concatenate([first * cos - second * sin, second * cos + first * sin], axis=-1)


def soft_cap(x, cap):
  """simply/model_lib.py:107-109: cap * tanh(x / cap); cap <= 0 disables
  (simply/model_lib.py:624, :3187)."""
  if cap is None or cap <= 0:
    return x
  c = x.dtype.type(cap)
  return c * np.tanh(x / c)


def attention_mask(q_pos, k_pos, window):
  """simply/model_lib.py:469-515 restated for one sequence: causal, and for a
  local layer at most `window` keys including the query itself (the
  reference's window_size excludes the query, simply/config_lib.py:874, so
  window = window_size + 1, simply/utils/ragged_paged_attention.py:922)."""
  q = np.asarray(q_pos)[:, None]
  k = np.asarray(k_pos)[None, :]
  mask = k <= q
  if window is not None:
    mask &= (q - k) < window
  return mask


def grouped_attention(q, k, v, q_pos, k_pos, logit_cap, window):
  """simply/model_lib.py:610-638 (scores -> soft cap -> mask by select -> softmax -> PV)
  with the grouping of simply/model_lib.py:2306-2310: query head n reads kv head n // G.

  q: [Tq, Hq, dh] (already rotated and scaled); k, v: [Tk, Hkv, dh].
  """
  dtype = q.dtype
  hq, hkv = q.shape[1], k.shape[1]
  group = hq // hkv
  mask = attention_mask(q_pos, k_pos, window)
  mask_value = dtype.type(-0.5 * np.finfo(np.float32).max)  # simply/utils/common.py:543-551
  out = np.zeros_like(q)
  for n in range(hq):
    m = n // group
    s = q[:, n, :] @ k[:, m, :].T
    s = soft_cap(s, logit_cap)
    s = np.where(mask, s, mask_value)
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p = p / p.sum(axis=-1, keepdims=True)
    out[:, n, :] = p @ v[:, m, :]
  return out


def gelu_tanh(x):
  """simply/model_lib.py:93-96."""
  dtype = x.dtype
  c = dtype.type(np.sqrt(2.0 / np.pi))
  return dtype.type(0.5) * x * (dtype.type(1.0) + np.tanh(c * (x + dtype.type(0.044715) * x ** 3)))


def gated_feed_forward(y, w_gate, w_up, w_down):
  """simply/model_lib.py:714-730: act(gate) * up, then down.  Weights are [out, in]."""
  return (gelu_tanh(y @ w_gate.T) * (y @ w_up.T)) @ w_down.T


def attention_layer(y, positions, w, cfg, layer, k_override=None):
  """simply/model_lib.py:2106-2110 (projections), :2010-2019 (rope, then q scale),
  :2362 (output projection).  Returns (output, (k, v)) so that a test can let
  another layer read this layer's keys and values."""
  hq, hkv, dh = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
  t = y.shape[0]
  q = (y @ w["q"].T).reshape(t, hq, dh)
  q = rope(q, positions, cfg["rope_theta"]) * y.dtype.type(cfg["query_pre_attn_scalar"] ** -0.5)
  if k_override is None:
    k = rope((y @ w["k"].T).reshape(t, hkv, dh), positions, cfg["rope_theta"])
    v = (y @ w["v"].T).reshape(t, hkv, dh)
  else:
    k, v = k_override
  window = cfg["sliding_window"] if layer_is_local(cfg, layer) else None
  o = grouped_attention(q, k, v, positions, positions, cfg["attn_logit_softcapping"], window)
  return o.reshape(t, hq * dh) @ w["o"].T, (k, v)


def layer_is_local(cfg, layer):
  """simply/model_lib.py:2839-2844 with block_attn_pattern=('local','global')
  (simply/config_lib.py:877-880): even layers are local."""
  types = cfg.get("layer_types")
  if types:
    return types[layer] == "sliding_attention"
  return layer % 2 == 0


def block(h, positions, w, cfg, layer):
  """simply/model_lib.py:2659-2708 with use_pre_ln, use_post_ln and no post-skip norm
  (simply/config_lib.py:868-870): the post norm acts on the branch before the add."""
  eps = cfg["rms_norm_eps"]
  a, _ = attention_layer(rms_norm(h, w["pre_attn"], eps), positions, w, cfg, layer)
  h = h + rms_norm(a, w["post_attn"], eps)
  f = gated_feed_forward(rms_norm(h, w["pre_ffn"], eps), w["gate"], w["up"], w["down"])
  return h + rms_norm(f, w["post_ffn"], eps)


def logits_from_hidden(h, final_scale, table, cfg):
  """simply/model_lib.py:3183-3188: final norm, tied table, final soft cap."""
  x = rms_norm(h, final_scale, cfg["rms_norm_eps"])
  return soft_cap(x @ np.asarray(table, h.dtype).T, cfg["final_logit_softcapping"])


# ----------------------------------------------------------------------------
# Whole model
# ----------------------------------------------------------------------------


def read_model_folder(model_dir, dtype=np.float32):
  """config.json as a dict and every tensor as a NumPy array of `dtype`."""
  from safetensors import safe_open

  with open(os.path.join(model_dir, "config.json")) as f:
    cfg = json.load(f)
  tensors = {}
  with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
    for name in f.keys():
      tensors[name] = f.get_tensor(name).float().numpy().astype(dtype, copy=False)
  return cfg, tensors


def layer_weights(tensors, i):
  p = f"model.layers.{i}."
  return {
      "q": tensors[p + "self_attn.q_proj.weight"],
      "k": tensors[p + "self_attn.k_proj.weight"],
      "v": tensors[p + "self_attn.v_proj.weight"],
      "o": tensors[p + "self_attn.o_proj.weight"],
      "gate": tensors[p + "mlp.gate_proj.weight"],
      "up": tensors[p + "mlp.up_proj.weight"],
      "down": tensors[p + "mlp.down_proj.weight"],
      "pre_attn": tensors[p + "input_layernorm.weight"],
      "post_attn": tensors[p + "post_attention_layernorm.weight"],
      "pre_ffn": tensors[p + "pre_feedforward_layernorm.weight"],
      "post_ffn": tensors[p + "post_feedforward_layernorm.weight"],
  }


class PlainGemma2:
  """The whole decoder on one sequence: tokens -> logits at every position."""

  def __init__(self, model_dir, dtype=np.float32):
    self.dtype = np.dtype(dtype).type
    self.cfg, self.tensors = read_model_folder(model_dir, dtype)

  def forward(self, tokens):
    """simply/model_lib.py:2935-3189 for one sequence at positions 0..T-1: [T, vocab]."""
    cfg, t = self.cfg, self.tensors
    positions = np.arange(len(tokens))
    h = embed(tokens, t["model.embed_tokens.weight"], self.dtype)
    for i in range(cfg["num_hidden_layers"]):
      h = block(h, positions, layer_weights(t, i), cfg, i)
    return logits_from_hidden(h, t["model.norm.weight"], t["model.embed_tokens.weight"], cfg)

  def greedy(self, prompt, steps):
    """temperature == 0 -> argmax (simply/utils/sampling_lib.py:494-497)."""
    tokens = list(prompt)
    for _ in range(steps):
      tokens.append(int(np.argmax(self.forward(tokens)[-1])))
    return tokens[len(prompt):]

  def sample(self, prompt, steps, temperature, seed, top_k=-1, top_p=1.0):
    tokens = list(prompt)
    for _ in range(steps):
      logits = self.forward(tokens)[-1].astype(np.float32)
      tokens.append(sample_token(logits, temperature, top_k, top_p, seed, len(tokens)))
    return tokens[len(prompt):]


# ----------------------------------------------------------------------------
# Sampling
# ----------------------------------------------------------------------------

_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK32 = np.uint64(0xFFFFFFFF)


def philox4x32(counter, key):
  """Philox-4x32 with 10 rounds (Salmon et al., 2011) on arrays of uint32 counters.

  counter: 4 arrays of equal shape; key: 2 Python ints.  Returns 4 uint32 arrays.
  """
  c = [np.asarray(x, np.uint64) & _MASK32 for x in counter]
  k0, k1 = key[0] & 0xFFFFFFFF, key[1] & 0xFFFFFFFF
  for _ in range(10):
    p0 = _M0 * c[0]
    p1 = _M1 * c[2]
    hi0, lo0 = p0 >> np.uint64(32), p0 & _MASK32
    hi1, lo1 = p1 >> np.uint64(32), p1 & _MASK32
    c = [hi1 ^ c[1] ^ np.uint64(k0), lo1, hi0 ^ c[3] ^ np.uint64(k1), lo0]
    k0 = (k0 + _W0) & 0xFFFFFFFF
    k1 = (k1 + _W1) & 0xFFFFFFFF
  return [x.astype(np.uint32) for x in c]


def gumbel_noise(vocab, seed, position):
  """Standard Gumbel noise for every vocabulary entry of one sampling event.

  The generator is keyed by the request's 64-bit seed; the counter is
  (entry // 4, position of the sampled token, 0, 0) and entry % 4 picks the word.
  """
  blocks = (vocab + 3) // 4
  idx = np.arange(blocks, dtype=np.uint64)
  zeros = np.zeros(blocks, np.uint64)
  words = philox4x32([idx, zeros + np.uint64(position), zeros, zeros],
                     (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
  bits = np.stack(words, axis=1).reshape(-1)[:vocab]
  u = ((bits >> np.uint32(8)).astype(np.float32) + np.float32(0.5)) * np.float32(2.0 ** -24)
  return -np.log(-np.log(u))


def top_k_mask(logits, top_k):
  """simply/utils/sampling_lib.py:427-431."""
  k = max(min(top_k, logits.shape[-1]), 1)
  order = np.argsort(-logits, kind="stable")[:k]
  mask = np.zeros(logits.shape, bool)
  mask[order] = True
  return mask


def top_p_mask(logits, top_p):
  """simply/utils/sampling_lib.py:434-441: keep sorted entries whose exclusive
  cumulative probability is below top_p."""
  z = logits - logits.max()
  probs = np.exp(z) / np.exp(z).sum()
  order = np.argsort(-logits, kind="stable")
  cum = np.concatenate([[0.0], np.cumsum(probs[order])])[:-1]
  mask = np.zeros(logits.shape, bool)
  mask[order[cum < top_p]] = True
  return mask


def token_logprob(logits, token, temperature, top_k, top_p):
  """simply/utils/sampling_lib.py:540-601: the log-probability of `token` under the distribution
  `sample_token` draws from: 0 for a greedy row (the token is the argmax); otherwise the
  log-softmax of logits / temperature over the entries that top-k and top-p keep."""
  logits = np.asarray(logits, np.float32)
  if temperature == 0 or top_k == 1:
    return 0.0 if int(np.argmax(logits)) == token else float("-inf")
  scaled = (logits / np.float32(temperature)).astype(np.float64)
  keep = np.ones(logits.shape, bool)
  if top_k > 0:
    keep &= top_k_mask(scaled.astype(np.float32), top_k)
  if top_p < 1.0:
    inner = np.where(keep, scaled, -np.inf).astype(np.float32)
    keep &= top_p_mask(inner, top_p)
  if not keep[token]:
    return float("-inf")
  kept = scaled[keep]
  return float(scaled[token] - kept.max() - np.log(np.exp(kept - kept.max()).sum()))


def sample_token(logits, temperature, top_k, top_p, seed, position):
  """simply/utils/sampling_lib.py:472-537: greedy when temperature == 0 or top_k == 1;
  otherwise logits / temperature, masked by top-k and top-p (top-p within the
  top-k candidates when both are set, :444-469), then a categorical draw.  The
  draw is Gumbel-max, as jax.random.categorical does (simply/utils/distributions.py:80-83),
  with this engine's own counter-based noise."""
  logits = np.asarray(logits, np.float32)
  if temperature == 0 or top_k == 1:
    return int(np.argmax(logits))
  scaled = logits / np.float32(temperature)
  keep = np.ones(logits.shape, bool)
  if top_k > 0:
    keep &= top_k_mask(scaled, top_k)
  if top_p < 1.0:
    inner = np.where(keep, scaled, -np.inf).astype(np.float32)
    keep &= top_p_mask(inner, top_p)
  noisy = np.where(keep, scaled + gumbel_noise(logits.shape[0], seed, position), -np.inf)
  return int(np.argmax(noisy))
