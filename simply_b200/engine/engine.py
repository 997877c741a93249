"""The engine: model + cache + step function, and generation on top of the scheduler.

`step_raw` is the one step function: it takes a batch of (request slot, its next
tokens, wanted places), makes room in the cache, runs exactly those tokens as
one ragged batch through the model and returns float32 logits at the wanted
places.  Generation (`generate`, `add_request` + `step`) and trace replay both
go through it.

Reference counterparts: `SamplingState.mixed_step`
(simply/utils/ragged_paged_attention.py:1954-2062) is one step; `Batcher.loop`
(simply/serving/page_batcher.py:701-895) and `LMInterface.generate`
(simply/model_lib.py:4662-4942) are the loops above it.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Sequence

import numpy as np
import torch

from simply_b200.cache.manager import CacheManager
from simply_b200.config import EngineConfig, load_config
from simply_b200.engine.batch import StepContext, StepEntry, pack_step
from simply_b200.engine.scheduler import Request, Scheduler, StepPlan
from simply_b200.parts.model import DecoderModel
from simply_b200.sampling.params import SamplingParams
from simply_b200.weights.loader import load_tensors
from simply_b200.weights.random_init import random_tensors

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


@dataclasses.dataclass
class GenerationResult:
  """What `generate` returns per prompt, after the reference's `SamplingOutput`
  (simply/model_lib.py:4459-4480): output tokens and whether the output was cut short."""

  request_id: object
  input_token_ids: list[int]
  output_token_ids: list[int]
  finish_reason: str
  num_preemptions: int = 0
  # With SamplingParams(logprobs=True): log-probability of every output token under the
  # distribution it was drawn from (the reference's `output_token_logprobs`).
  output_token_logprobs: list[float] | None = None

  @property
  def is_truncated(self) -> bool:
    return self.finish_reason != "eos"


def _derived_seed(n: int) -> int:
  """The n-th of a fixed sequence of well-mixed 64-bit seeds (splitmix64)."""
  z = (0x9E3779B97F4A7C15 * (n + 1)) & 0xFFFFFFFFFFFFFFFF
  z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
  z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
  return z ^ (z >> 31)


def default_ops(dtype: torch.dtype):
  """The CUDA kernel table; fails loudly when there is no GPU or the extension cannot be built."""
  from simply_b200.kernels.ops import CudaOps
  return CudaOps(dtype)


class Engine:

  def __init__(self, config: Any, tensors: dict[str, torch.Tensor],
               engine_config: EngineConfig | None = None, *, ops: Any = None,
               device: torch.device | str | None = None):
    self.config = config
    spec = config.model_spec()
    self.engine_config = (engine_config or EngineConfig()).resolved(spec.max_context)
    self.dtype = _TORCH_DTYPE[self.engine_config.activation_dtype]
    self.ops = ops if ops is not None else default_ops(self.dtype)
    if device is None:
      device = "cuda" if ops is None else next(iter(tensors.values())).device
    self.device = torch.device(device)
    self.model = DecoderModel(spec)
    self.model.bind(tensors, self.ops)
    ec = self.engine_config
    self.cache = CacheManager(
        self.model.cache_needs(), page_size=ec.page_size, max_slots=ec.batch_size,
        max_seq_len=ec.max_seq_len, max_cache_tokens=ec.max_cache_tokens, dtype=self.dtype,
        device=self.device, poison_freed_pages=ec.poison_freed_pages,
        step_tokens=None if ec.max_window_cache_tokens < 0 else ec.max_num_issue_tokens,
        burst_tokens=min(max(ec.intermediate_steps, 1), 64),
        windowed_cache_tokens=max(ec.max_window_cache_tokens, 0))
    self.caches = {**self.cache.paged, **self.cache.states}
    eos = getattr(config, "eos_token_id", None)
    eos_ids = () if eos is None else (tuple(eos) if isinstance(eos, (tuple, list)) else (eos,))
    self.scheduler = Scheduler(self.cache, max_num_issue_tokens=ec.max_num_issue_tokens,
                               max_seq_len=ec.max_seq_len, eos_ids=eos_ids)
    self._next_id = 0
    self._unseeded = 0  # requests that came without a sampling seed so far
    self._burst_params = None  # sampling words of the last decode burst's requests
    self.num_steps = 0
    self._decode_runner = None
    if ec.use_cuda_graphs and self.device.type == "cuda" and hasattr(self.ops, "decode_advance"):
      from simply_b200.engine import decode_graph
      if decode_graph.graphable(self.model):
        self._decode_runner = decode_graph.DecodeRunner(self)

  # ---- construction ---------------------------------------------------------
  @classmethod
  def from_folder(cls, model_dir: str, engine_config: EngineConfig | None = None, *,
                  ops: Any = None, device: torch.device | str | None = None) -> "Engine":
    """A model folder (config.json + *.safetensors) -> engine."""
    config = load_config(model_dir)
    ec = engine_config or EngineConfig()
    dtype = _TORCH_DTYPE[ec.activation_dtype]
    if device is None:
      device = "cuda" if ops is None else "cpu"
    if ops is None:
      ops = default_ops(dtype)
    tensors = load_tensors(model_dir, DecoderModel(config.model_spec()).tensor_specs(), dtype, device,
                           keep_float32=ec.keep_float32_weights)
    return cls(config, tensors, ec, ops=ops, device=device)

  @classmethod
  def from_config(cls, config: Any, seed: int, engine_config: EngineConfig | None = None, *,
                  matrix_std: float = 0.02, scale_std: float = 0.0, ops: Any = None,
                  device: torch.device | str | None = None) -> "Engine":
    """Random weights drawn on the device, without a model folder in between."""
    ec = engine_config or EngineConfig()
    dtype = _TORCH_DTYPE[ec.activation_dtype]
    if device is None:
      device = "cuda" if ops is None else "cpu"
    if ops is None:
      ops = default_ops(dtype)
    tensors = random_tensors(DecoderModel(config.model_spec()).tensor_specs(), seed,
                             matrix_std=matrix_std, scale_std=scale_std, dtype=dtype, device=device)
    return cls(config, tensors, ec, ops=ops, device=device)

  # ---- the step function ------------------------------------------------------
  def open_request(self, owner: object = None) -> int:
    """Takes a slot for a request that will be stepped by hand (replay); returns the slot."""
    return self.cache.acquire_slot(owner if owner is not None else object())

  def close_request(self, slot: int) -> None:
    self.cache.release_slot(slot)

  def step_raw(self, entries: Sequence[StepEntry], *, from_graph: bool = False) -> torch.Tensor | None:
    """Runs one batch; returns float32 logits [wanted, vocab] (None if nothing is wanted).

    `from_graph=True` lets a step in which every entry brings one token run the way generation
    runs such steps, as a replay of the decode graph (when the engine has graphs at all and keeps
    their logits); the tokens the graph samples on the way are dropped."""
    runner = self._decode_runner
    if (from_graph and runner is not None and runner.keep_logits
        and all(len(e.tokens) == 1 for e in entries)):
      return self._step_raw_from_graph(entries)
    ctx = self._prepare(entries)
    hold = getattr(self.ops, "hold_stream", None)  # (a kernel table without streams has none)
    if hold is None:
      logits = self.model.forward(ctx, self.caches)
    else:
      with hold():
        logits = self.model.forward(ctx, self.caches)
    self.num_steps += 1
    return logits

  def _step_raw_from_graph(self, entries: Sequence[StepEntry]) -> torch.Tensor | None:
    self._check_token_ids([np.asarray(e.tokens) for e in entries])
    for i, e in enumerate(entries):
      if any(w != 0 for w in e.want):
        raise ValueError(f"entry {i}: wanted place outside its 1 token")
    lengths = [self.cache.length(e.slot) + 1 for e in entries]
    params = self.ops.pack_sample_params([0.0] * len(entries), [-1] * len(entries), [1.0] * len(entries),
                                         [0] * len(entries), lengths)
    self._decode_runner.run([e.slot for e in entries], [int(e.tokens[0]) for e in entries], params, 1)
    rows = [i for i, e in enumerate(entries) if len(e.want)]
    if not rows:
      return None
    return self._decode_runner.last_logits[0][rows]

  def _check_token_ids(self, token_arrays) -> None:
    vocab = self.model.spec.vocab_size
    for ids in token_arrays:
      if ids.size and (ids.min() < 0 or ids.max() >= vocab):
        bad = ids[(ids < 0) | (ids >= vocab)][0]
        raise ValueError(f"token id {bad} is outside the vocabulary of {vocab}")

  def _prepare(self, entries: Sequence[StepEntry]) -> StepContext:
    token_arrays = [np.asarray(e.tokens) for e in entries]
    self._check_token_ids(token_arrays)
    lengths = [self.cache.length(e.slot) for e in entries]
    self.cache.extend([(e.slot, len(e.tokens)) for e in entries])
    ctx = pack_step(entries, lengths, [g.tables for g in self.cache.groups],
                    self.cache.page_size, self.ops, self.device, token_arrays)
    ctx.older_keys_settled = True  # what the cache holds below a request's length comes from earlier steps
    return ctx

  # ---- generation -------------------------------------------------------------
  def add_request(self, prompt: Sequence[int], params: SamplingParams | None = None,
                  request_id: object = None) -> Request:
    if request_id is None:
      request_id = self._next_id
      self._next_id += 1
    params = params or SamplingParams()
    if params.seed is None:
      # No seed given: one per request, from the order of arrival, so that equal prompts draw
      # different samples (a run of the same requests in the same order still repeats itself).
      params = dataclasses.replace(params, seed=_derived_seed(self._unseeded))
      self._unseeded += 1
    return self.scheduler.add(request_id, prompt, params)

  def cancel(self, request_id: object) -> bool:
    return self.scheduler.cancel(request_id)

  def has_unfinished(self) -> bool:
    return self.scheduler.has_unfinished()

  def step(self) -> list[Request]:
    """Schedules, runs and samples one step; returns the requests that ended in it."""
    plan = self.scheduler.schedule()
    finished = list(plan.failed)
    if not plan.entries:
      return finished
    if self._decode_runner is not None and all(e.request.is_decoding for e in plan.entries):
      return finished + self._decode_burst(plan)
    entries = []
    samplers = []
    for e in plan.entries:
      r = e.request
      toks = r.tokens[r.num_cached:r.num_cached + e.num_tokens]
      entries.append(StepEntry(r.slot, toks, (e.num_tokens - 1,) if e.samples else ()))
      if e.samples:
        samplers.append(r)
    logits = self.step_raw(entries)
    sampled: dict[object, int] = {}
    logprobs: dict[object, float] | None = None
    if samplers:
      want_logprobs = any(r.params.logprobs for r in samplers)
      tokens = self.ops.sample(
          logits,
          [r.params.temperature for r in samplers],
          [r.params.top_k for r in samplers],
          [r.params.top_p for r in samplers],
          [r.params.seed for r in samplers],
          [len(r.tokens) for r in samplers], **({"logprobs": True} if want_logprobs else {}))
      if want_logprobs:
        tokens, lp = tokens
        logprobs = {r.request_id: v for r, v in zip(samplers, lp.tolist())}
      for r, t in zip(samplers, tokens.tolist()):
        sampled[r.request_id] = t
    return finished + self.scheduler.commit(plan, sampled, logprobs)

  def _decode_burst(self, plan: StepPlan) -> list[Request]:
    """A step (or `intermediate_steps` steps in a row) in which every entry decodes one token,
    replayed from a CUDA graph."""
    requests = [e.request for e in plan.entries]
    steps = max(1, min(self.engine_config.intermediate_steps, self._decode_runner.MAX_BURST))
    for r in requests:
      steps = min(steps, r.params.max_decode_steps - r.num_output,
                  self.engine_config.max_seq_len - len(r.tokens))
    steps = max(steps, 1)
    while steps > 1 and self.cache.pages_short([(r.slot, steps) for r in requests]):
      steps //= 2
    # The sampling words of a batch change only in the position to sample: the rest is kept from
    # the last burst of the same requests.
    key = tuple(id(r) for r in requests)
    if self._burst_params is not None and self._burst_params[0] == key:
      params = self._burst_params[1].copy()
      params[:, 5] = [len(r.tokens) for r in requests]
    else:
      params = self.ops.pack_sample_params(
          [r.params.temperature for r in requests], [r.params.top_k for r in requests],
          [r.params.top_p for r in requests], [r.params.seed for r in requests],
          [len(r.tokens) for r in requests])
      self._burst_params = (key, params, requests)  # (the requests are held so that their ids stay theirs)
    want_logprobs = any(r.params.logprobs for r in requests)
    tokens = self._decode_runner.run([r.slot for r in requests], [r.tokens[-1] for r in requests],
                                     params, steps, logprobs=want_logprobs)
    lp_rows = self._decode_runner.last_logprobs if want_logprobs else None
    finished: list[Request] = []
    for i in range(steps):
      row = tokens[i].tolist()
      live = [(j, e) for j, e in enumerate(plan.entries) if e.request.status.value == "running"]
      step_plan = StepPlan([e for _, e in live], [], [])
      sampled = {e.request.request_id: row[j] for j, e in live}
      logprobs = None
      if lp_rows is not None:
        lp = lp_rows[i].tolist()
        logprobs = {e.request.request_id: lp[j] for j, e in live}
      finished += self.scheduler.commit(step_plan, sampled, logprobs)
    # Requests that are still live hold exactly the tokens the burst cached.
    return finished

  def score_tokens(self, tokens: Sequence[int], params: SamplingParams | None = None,
                   rows_per_step: int = 256) -> list[float]:
    """The log-likelihood of every token but the first, given the tokens before it: len(tokens) - 1
    values (the reference's `LMInterface.score_tokens`, simply/model_lib.py:4995-5036).  `params`
    gives the temperature, top-k and top-p under which a token is scored (default: the plain
    softmax); a greedy setting scores the most likely token 0 and any other -inf.  The tokens run
    through the step function in portions of `rows_per_step`, in a slot of their own."""
    params = params or SamplingParams(temperature=1.0)
    tokens = [int(t) for t in tokens]
    if len(tokens) < 2:
      return []
    if len(tokens) - 1 > self.engine_config.max_seq_len:
      raise ValueError(f"{len(tokens)} tokens exceed max_seq_len {self.engine_config.max_seq_len}")
    slot = self.open_request(("score", id(tokens)))
    scores: list[float] = []
    try:
      for start in range(0, len(tokens) - 1, rows_per_step):
        portion = tokens[start:min(start + rows_per_step, len(tokens) - 1)]
        logits = self.step_raw([StepEntry(slot, portion, tuple(range(len(portion))))])
        targets = torch.tensor(tokens[start + 1:start + 1 + len(portion)], dtype=torch.int32)
        scores += self.ops.token_logprobs(logits, targets, params.temperature, params.top_k, params.top_p).tolist()
    finally:
      self.close_request(slot)
    return scores

  def generate_text(self, prompts: Sequence[str], params: SamplingParams | None = None, *,
                    processor: Any) -> list[tuple[str, GenerationResult]]:
    """Text in, text out (the reference's `LMInterface.generate` with `input_text`,
    simply/model_lib.py:4662-4717): `processor` (simply_b200.text.TextProcessor) puts the bos id
    in front of each encoded prompt and names the eos ids, which end a request unless `params`
    names stop tokens of its own.  Returns (generated text, result) per prompt; the text leaves
    out the token that ended the request."""
    params = params or SamplingParams()
    if params.stop_token_ids is None:
      params = dataclasses.replace(params, stop_token_ids=tuple(processor.eos_ids))
    results = self.generate([processor.encode(p) for p in prompts], params)
    out = []
    for r in results:
      ids = r.output_token_ids
      if r.finish_reason == "eos" and ids:
        ids = ids[:-1]
      out.append((processor.decode(ids), r))
    return out

  def generate(self, prompts: Sequence[Sequence[int]],
               params: SamplingParams | Sequence[SamplingParams] | None = None
               ) -> list[GenerationResult]:
    """Generates for every prompt (token ids in, token ids out), batching them continuously."""
    if params is None or isinstance(params, SamplingParams):
      params = [params or SamplingParams()] * len(prompts)
    if len(params) != len(prompts):
      raise ValueError(f"{len(prompts)} prompts but {len(params)} sampling parameter sets")
    requests = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
    while self.has_unfinished():
      self.step()
    return [GenerationResult(r.request_id, r.prompt, r.output, r.finish_reason, r.num_preemptions,
                             list(r.logprobs) if r.params.logprobs else None)
            for r in requests]
