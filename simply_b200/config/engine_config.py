"""Engine settings that are not part of the model: cache pool, batch limits, dtype.

Names follow the reference's serving flags where it has them
(simply/serving/common_flags.py:19-132): `page_size` (:80), `batch_size` (:48)
is the number of requests that may be live at once, `max_seq_len` (:62) the
longest sequence a request may reach, `max_num_issue_tokens` (:92) the token
budget of one step, `activation_dtype` (:52).
"""

from __future__ import annotations

import dataclasses

_DTYPES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}


@dataclasses.dataclass(frozen=True)
class EngineConfig:
  activation_dtype: str = "bfloat16"
  # Tokens per cache page.
  page_size: int = 64
  # Requests that may be live at the same time (slots).
  batch_size: int = 8
  # Longest sequence (prompt + generated) of one request; 0 means the model's
  # max_position_embeddings.
  max_seq_len: int = 0
  # Tokens the cache pool can hold over all live requests: a group of layers that keeps every
  # token gets ceil(max_cache_tokens / page_size) pages.  0 means batch_size * max_seq_len.
  max_cache_tokens: int = 0
  # Tokens the pool of a group of sliding-window layers holds.  0 sizes it from the window: what
  # batch_size requests can hold at once when a step brings at most max_num_issue_tokens prompt
  # tokens (the reference's local_total_num_pages beside global_total_num_pages,
  # simply/serving/page_server.py:175-196); -1 makes it as large as max_cache_tokens, for callers
  # of `step_raw` that bring longer portions than max_num_issue_tokens.
  max_window_cache_tokens: int = 0
  # Token budget of one step (decoded tokens and prompt portions together);
  # 0 means 2048.
  max_num_issue_tokens: int = 0
  # In bfloat16, keep matrices that the model folder stores in 32 bits as they are (twice the
  # memory, products on the 32-bit kernel) instead of narrowing them to the activation dtype.
  keep_float32_weights: bool = False
  # Replay decode-only steps from CUDA graphs.
  use_cuda_graphs: bool = True
  # Decode steps that run in a row without the host in between (the reference's flag of
  # the same name, simply/serving/common_flags.py:84-86); a request that ends inside such a
  # burst drops the tokens sampled after its end.  At most 64.
  intermediate_steps: int = 1
  # Fill freed pages with NaN so that a read of a page the request does not own shows.
  poison_freed_pages: bool = False

  def __post_init__(self):
    if self.activation_dtype not in _DTYPES:
      raise ValueError(
          f"activation_dtype must be one of {sorted(set(_DTYPES.values()))}, "
          f"got {self.activation_dtype!r}")
    object.__setattr__(self, "activation_dtype", _DTYPES[self.activation_dtype])
    if self.page_size <= 0:
      raise ValueError(f"page_size must be positive, got {self.page_size}")
    if self.batch_size <= 0:
      raise ValueError(f"batch_size must be positive, got {self.batch_size}")
    for k in ("max_seq_len", "max_cache_tokens", "max_num_issue_tokens"):
      if getattr(self, k) < 0:
        raise ValueError(f"{k} must be >= 0, got {getattr(self, k)}")
    if self.max_window_cache_tokens < -1:
      raise ValueError(f"max_window_cache_tokens must be >= -1, got {self.max_window_cache_tokens}")

  def resolved(self, model_max_context: int) -> "EngineConfig":
    """Fills the zero defaults from the model's longest context."""
    max_seq_len = self.max_seq_len or model_max_context
    if max_seq_len > model_max_context:
      raise ValueError(
          f"max_seq_len {max_seq_len} exceeds the model's max_position_embeddings "
          f"{model_max_context}")
    return dataclasses.replace(
        self,
        max_seq_len=max_seq_len,
        max_cache_tokens=self.max_cache_tokens or self.batch_size * _round_up(max_seq_len, self.page_size),
        max_num_issue_tokens=self.max_num_issue_tokens or 2048,
    )


def _round_up(n: int, m: int) -> int:
  return (n + m - 1) // m * m
