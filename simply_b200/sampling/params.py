"""Sampling parameters of one request.

Field names and meanings follow the reference's `SamplingParams`
(simply/utils/sampling_lib.py:73-100) and serving flags
(simply/serving/common_flags.py:76-84): `temperature` (0 means greedy,
sampling_lib.py:494-497), `top_k` (-1 = whole vocabulary; 1 means greedy),
`top_p` (1.0 = off), `max_decode_steps`.  `seed` is this engine's: every request
draws from its own counter-based generator, keyed by (seed, position of the
sampled token), so its tokens do not depend on what else is in the batch (the
reference splits one global key per step, simply/utils/ragged_paged_attention.py:2031,
which also makes the rows of a batch independent of each other).  A request
given an explicit seed is reproducible: the same prompt, parameters and seed
give the same tokens, in any batch.  With `seed=None` (the default) the engine
derives a seed from the order in which it received the request, so that two
requests with the same prompt draw different samples, as rows of the
reference's batch do; `logprobs=True` also returns the log-probability of each
emitted token (simply/utils/sampling_lib.py:540-601).
"""

from __future__ import annotations

import dataclasses


@dataclasses.dataclass(frozen=True)
class SamplingParams:
  temperature: float = 1.0
  top_k: int = -1
  top_p: float = 1.0
  max_decode_steps: int = 256
  seed: int | None = None
  # Token ids that end the request when sampled; None means the model's eos ids.
  stop_token_ids: tuple[int, ...] | None = None
  # Also return the log-probability of every emitted token (0 for greedy requests).
  logprobs: bool = False

  def __post_init__(self):
    if self.temperature < 0:
      raise ValueError(f"temperature must be >= 0, got {self.temperature}")
    if self.top_k == 0 or self.top_k < -1:
      raise ValueError(f"top_k must be -1 (off) or positive, got {self.top_k}")
    if not 0.0 < self.top_p <= 1.0:
      raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
    if self.max_decode_steps <= 0:
      raise ValueError(f"max_decode_steps must be positive, got {self.max_decode_steps}")

  @property
  def greedy(self) -> bool:
    return self.temperature == 0 or self.top_k == 1
