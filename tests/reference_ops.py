"""Plain PyTorch statement of every kernel of the engine's kernel table.

Two uses.  The GPU tests call one CUDA kernel and the function of the same
name here on the same inputs.  The CPU tests hand an instance to the engine in
place of the CUDA table, so that the cache manager, the step function, the
scheduler and replay can be checked against the plain NumPy model on a machine
without a GPU.  Nothing in the package imports this file.

Every function computes in float32 (float64 where noted) from inputs of the
activation dtype and rounds once at the end, as the kernels do.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from tests.plain import gemma2_plain as plain


class ReferenceOps:

  def __init__(self, dtype: torch.dtype = torch.float32):
    self.dtype = dtype
    self.name = "reference"

  # ---- checks ---------------------------------------------------------------
  def check_attention(self, head_dim, num_heads, num_kv_heads):
    pass

  # ---- dense ----------------------------------------------------------------
  def linear(self, x, w):
    return (x.float() @ w.float().t()).to(self.dtype)

  def gated_linear(self, x, w_gate_up, activation):
    return self.gated_activation(self.linear(x, w_gate_up), activation)

  def cast(self, x, dtype):
    return x.to(dtype)

  def check_errors(self):
    pass

  def embed(self, table, ids, scale):
    s = torch.tensor(scale, dtype=torch.float32)
    if table.dtype == torch.bfloat16:
      s = s.to(torch.bfloat16).float()
    return table[ids.long()].float() * s

  def lm_head(self, x, table, cap):
    logits = x.float() @ table.float().t()
    if cap > 0:
      logits = cap * torch.tanh(logits / cap)
    return logits

  def gated_activation(self, gate_up, activation):
    f = gate_up.shape[1] // 2
    g, u = gate_up[:, :f].float(), gate_up[:, f:].float()
    if activation == 0:
      a = 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3)))
    elif activation == 1:
      a = g * torch.sigmoid(g)
    elif activation == 2:
      a = torch.relu(g)
    else:
      raise ValueError(f"unknown activation code {activation}")
    return (a * u).to(self.dtype)

  # ---- norms ----------------------------------------------------------------
  @staticmethod
  def _rms(x, w, eps, plus_one):
    x = x.float()
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y * (w.float() + 1.0 if plus_one else w.float())

  def rms_norm(self, x, w, eps, plus_one):
    return self._rms(x, w, eps, plus_one).to(self.dtype)

  def residual_norm(self, h, branch, post, pre, rows):
    if rows is not None:
      idx = rows.long()
      h = h[idx].clone()
      branch = branch[idx] if branch is not None else None
    if branch is not None:
      b = self._rms(branch, post.weight, post.eps, post.plus_one) if post is not None else branch.float()
      h += b
    if pre is None:
      return None
    return self._rms(h, pre.weight, pre.eps, pre.plus_one).to(self.dtype)

  def gather_rows(self, x, rows):
    return x[rows.long()].clone()

  def add_to_residual(self, h, x):
    h += x.float()

  # ---- positions ------------------------------------------------------------
  def rotation_tables(self, positions, timescale, scale_factor):
    angle = positions.float()[:, None] / timescale[None, :] / np.float32(scale_factor)
    return torch.cos(angle), torch.sin(angle)

  def project_rotate_store(self, x, w_qkv, tables, q_scale, num_heads, num_kv_heads, head_dim, storage,
                           block_table, ctx):
    return self.rope_and_cache_write(self.linear(x, w_qkv), tables, q_scale, num_heads, num_kv_heads, head_dim,
                                     storage, block_table, ctx)

  def rope_and_cache_write(self, qkv, tables, q_scale, num_heads, num_kv_heads, head_dim, storage,
                           block_table, ctx):
    t = qkv.shape[0]
    nq = num_heads * head_dim
    nk = num_kv_heads * head_dim
    q = qkv[:, :nq].float().reshape(t, num_heads, head_dim)

    def rotate(x):
      if tables is None:
        return x
      cos, sin = tables[0][:, None, :], tables[1][:, None, :]
      half = head_dim // 2
      a, b = x[..., :half], x[..., half:]
      return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)

    q = (rotate(q) * np.float32(q_scale)).to(self.dtype)
    if storage is not None:
      k = rotate(qkv[:, nq:nq + nk].float().reshape(t, num_kv_heads, head_dim)).to(storage.dtype)
      v = qkv[:, nq + nk:nq + 2 * nk].reshape(t, num_kv_heads, head_dim).to(storage.dtype)
      pos = ctx.positions.long()
      page = block_table[ctx.token_seq.long(), pos // ctx.page_size].long()
      assert (page >= 0).all(), "a token would be written to a page its request does not hold"
      off = pos % ctx.page_size
      storage[page, 0, :, off, :] = k
      storage[page, 1, :, off, :] = v
    return q

  # ---- attention ------------------------------------------------------------
  def paged_attention(self, q, storage, block_table, ctx, *, num_heads, num_kv_heads, head_dim,
                      logit_softcap, window):
    t = q.shape[0]
    out = torch.zeros(t, num_heads, head_dim, dtype=torch.float32, device=q.device)
    group = num_heads // num_kv_heads
    cu_q = ctx.host["cu_q"]
    q_start = ctx.host["q_start"]
    ps = ctx.page_size
    for b in range(ctx.num_seqs):
      r0, r1 = int(cu_q[b]), int(cu_q[b + 1])
      kv_len = int(q_start[b]) + (r1 - r0)
      q_pos = torch.arange(int(q_start[b]), kv_len, device=q.device)
      lo = 0 if window is None else max(int(q_start[b]) - window + 1, 0)
      k_pos = torch.arange(lo, kv_len, device=q.device)
      page = block_table[b, (k_pos // ps)].long()
      assert (page >= 0).all(), "attention would read a page the request does not hold"
      kv = storage[page, :, :, k_pos % ps, :].float()  # [Tk, 2, Hkv, dh]
      mask = k_pos[None, :] <= q_pos[:, None]
      if window is not None:
        mask &= (q_pos[:, None] - k_pos[None, :]) < window
      for n in range(num_heads):
        m = n // group
        s = q[r0:r1, n, :].float() @ kv[:, 0, m, :].t()
        if logit_softcap > 0:
          s = logit_softcap * torch.tanh(s / logit_softcap)
        s = torch.where(mask, s, torch.tensor(-0.5 * torch.finfo(torch.float32).max, device=q.device))
        p = torch.softmax(s, dim=-1)
        out[r0:r1, n, :] = p @ kv[:, 1, m, :]
    return out.reshape(t, num_heads * head_dim).to(self.dtype)

  # ---- sampling -------------------------------------------------------------
  def token_logprobs(self, logits, tokens, temperature, top_k, top_p):
    rows = [logits[i].float().cpu().numpy() for i in range(logits.shape[0])]
    lp = [plain.token_logprob(rows[i], int(tokens[i]), float(temperature), int(top_k), float(top_p))
          for i in range(len(rows))]
    return torch.tensor(lp, dtype=torch.float32, device=logits.device)

  def sample(self, logits, temperature, top_k, top_p, seed, position, logprobs=False):
    """logits f32 [R, V]; the other arguments are host sequences of length R."""
    rows = [logits[i].float().cpu().numpy() for i in range(logits.shape[0])]
    out = [
        plain.sample_token(rows[i], float(temperature[i]), int(top_k[i]), float(top_p[i]), int(seed[i]),
                           int(position[i]))
        for i in range(logits.shape[0])
    ]
    tokens = torch.tensor(out, dtype=torch.int32, device=logits.device)
    if not logprobs:
      return tokens
    lp = [plain.token_logprob(rows[i], out[i], float(temperature[i]), int(top_k[i]), float(top_p[i]))
          for i in range(logits.shape[0])]
    return tokens, torch.tensor(lp, dtype=torch.float32, device=logits.device)
