"""The kernel table: every device operation the engine's parts call.

`CudaOps(dtype)` is the only implementation in the package.  It needs a CUDA
device and the compiled library and raises if either is missing; there is no
CPU path.  `dtype` is the activation and cache dtype: `torch.bfloat16` is the
serving path, `torch.float32` runs the whole model in true 32-bit arithmetic on
CUDA cores (own SIMT matrix product, no tensor-core mode).

Matrix products: in bfloat16, steps with at most 16 tokens use the engine's own
weight-streaming kernel (with fused soft-cap or gated-activation epilogues);
larger ones go to the library product (cuBLAS through torch.mm), as the
reference leaves them to XLA.  Everything else (attention over the paged cache,
norms, rotation, cache write, activation, embedding, sampling) is hand-written.
"""

from __future__ import annotations

import ctypes
import os
from typing import Any, Sequence

import numpy as np
import torch

from simply_b200.kernels import build

_F32, _BF16 = 0, 1
_ERRORS = {
    1: "a block-table entry outside the page pool was about to be followed",
    2: "a token id outside the embedding table",
    4: "a gather row outside the batch",
    8: "a wait for a bulk copy timed out",
}
_STATUS = {
    -2: "row too wide for the norm kernel's shared-memory buffer",
    -3: "unsupported cast",
    -4: "head size must be even",
    -5: "unknown activation code",
    -6: "too many rows for one launch of the float32 product",
    -7: "head size outside the attention kernel's range",
    -8: "query heads are no multiple of key/value heads",
    -9: "shape outside the weight-streaming product's range",
    -10: "batch outside the decode-advance kernel's range",
    -11: "head size does not allow a tensor map",
    -12: "the driver refused to encode a tensor map",
}


def _code(t: torch.Tensor) -> int:
  if t.dtype == torch.float32:
    return _F32
  if t.dtype == torch.bfloat16:
    return _BF16
  raise TypeError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t: torch.Tensor | None):
  """The tensor's address as the plain integer that a declared `c_void_p` parameter takes (every
  entry point's parameter types are declared; None is the null pointer)."""
  return None if t is None else t.data_ptr()


class KernelError(RuntimeError):
  pass


class _HeldStream:

  def __init__(self, ops):
    self.ops = ops

  def __enter__(self):
    self.previous = self.ops._step_stream
    self.ops._step_stream = ctypes.c_void_p(torch.cuda.current_stream(self.ops.device).cuda_stream)

  def __exit__(self, *exc):
    self.ops._step_stream = self.previous


class AttentionGraphPlan:
  """Static work list of the split-key attention kernel for decode bursts replayed from a CUDA
  graph, for one kind of attention layer (see `Mixer.graph_plans` for the interface).

  Every sequence gets the same number of work items, so the launch has a fixed size: the chunks
  that hold keys between the lowest key visible at the burst's first step and the highest at its
  last, then fillers.  The words are: items [batch * per_seq, 2], split_start [batch],
  split_count [batch]."""

  def __init__(self, ops: "CudaOps", window: int | None, group: int, num_kv_heads: int, head_dim: int,
               batch: int, bucket: int, max_burst: int, page_size: int):
    self.key = ops._plan_key(window, group, num_kv_heads, head_dim, page_size)
    self.window, self.group, self.batch = window, group, batch
    # Most keys a sequence of this bucket sees in such a layer during a burst.
    span = min(bucket, window + max_burst + 64) if window else bucket
    self.chunk = ops.decode_chunk_for([bucket - span] * batch, [bucket] * batch, num_kv_heads, head_dim)
    self.per_seq = -(-span // self.chunk) + 1
    self.words = batch * self.per_seq * 2 + 2 * batch

  def bind(self, view: torch.Tensor) -> dict:
    n = self.batch * self.per_seq * 2
    return dict(num_prefill=0, num_decode=self.batch * self.per_seq, chunk=self.chunk, rows_max=self.group,
                rows_per_tile=64, prefill_items=None, decode_items=view[:n],
                split_start=view[n:n + self.batch], split_count=view[n + self.batch:])

  def fill(self, host_words: np.ndarray, lengths: np.ndarray, steps: int) -> None:
    items, start, count = CudaOps.static_decode_plan(lengths, steps, self.window, self.chunk, self.per_seq)
    n = items.size
    host_words[:n] = items.reshape(-1)
    host_words[n:n + self.batch] = start
    host_words[n + self.batch:] = count

  def ranges(self, lengths: np.ndarray, steps: int):
    return CudaOps.decode_chunk_range(lengths, steps, self.window, self.chunk)


class CudaOps:

  name = "cuda"
  # Largest token count the weight-streaming product for a handful of tokens takes, and the largest
  # the one for a serving batch takes (csrc/gemm_skinny_bf16.cu, csrc/gemm_stream_tc.cu).
  skinny_max_rows = 16
  mid_max_rows = 128

  def __init__(self, dtype: torch.dtype = torch.bfloat16, device: str | torch.device = "cuda"):
    if dtype not in (torch.float32, torch.bfloat16):
      raise TypeError(f"activation dtype must be float32 or bfloat16, got {dtype}")
    if not torch.cuda.is_available():
      raise KernelError("simply_b200 needs a CUDA device (sm_100a); there is no CPU path")
    self.dtype = dtype
    self.device = torch.device(device)
    self.lib = build.load()
    major, minor = torch.cuda.get_device_capability(self.device)
    if major != 10:
      raise KernelError(f"kernels are built for sm_100a; this device is sm_{major}{minor}")
    self._declare()
    self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
    self._attn_fns: dict[int, tuple] = {}
    self._tensor_maps: dict[tuple, tuple] = {}
    # Work counter of the split-key attention kernel: zero between launches (its merge kernel resets it).
    self._attn_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
    # bfloat16 attention runs on tensor cores where the shape allows; False forces the general kernel.
    self.tensor_core_attention = True
    # Split-key attention: the chunk length is chosen so that the work items fill the kernel's
    # persistent grid evenly; decode_chunk > 0 fixes it instead (a multiple of 64).
    self.decode_chunk = 0
    self._decode_slots: dict[int, int] = {}
    # 0: the kernel is picked by the number of query rows; 1 forbids TMA; 16 forces the 16-row kernel (tests).
    self.decode_variant = 0
    self.direct_library_products = True  # False: through torch.mm
    self._library_workspaces: dict = {}
    self._step_stream = None
    # 0: prefill tiles of 64 query rows; 64 or 128 forces a size.
    self.prefill_rows = 0
    # Prefill attention on the tcgen05 tensor cores where the shapes allow (head size a multiple of
    # 64, group dividing 128, page size a power of two); False keeps the mma.sync kernel.
    self.prefill_tcgen05 = True
    # ... and there by pairs of blocks (cta_group::2) where the shapes allow (head size 128 or 256,
    # pages of at least 64 tokens); False keeps single blocks (tests).
    self.prefill_pairs = True
    self._rounded_scales: dict[float, float] = {}
    self.prefill_single_key_group = False  # True: 64-row tiles with 4 warps instead of 4 x 2 (experiments, tests)
    # 0: the weight-streaming product picks its warps per block; 4, 8 or 16 forces them (experiments).
    self.skinny_warps = 0
    # False keeps the q, k, v projection and the rotation + cache write as two kernels (tests).
    self.fused_qkv_rope = True
    # False sends steps of 17 to 64 tokens to the library product (tests, experiments); mid_split
    # fixes the number of blocks that share a row tile's k (0: the launch chooses).
    self.mid_rows_kernel = True
    # Most rows for which each kind of product takes that kernel rather than the library's: the
    # fused q, k, v projection, the gated product, a plain product, the output layer.  The kernel
    # takes up to 128 rows; measured inside decode steps of the Gemma 2 2B shape it is ahead of
    # the library's products up to 32 rows (by 1 to 2 % of the step) and behind them from 33
    # (by 1 to 4 %), so that is where the line is drawn.
    # From this many tokens the gated feed-forward product runs on the engine's own tcgen05 kernel
    # with the activation on the accumulators (csrc/gemm_gated_tc.cu); below, and for shapes it
    # does not take, the library's product and a pass of its own for the activation.  0: never.
    self.gated_tc_min_rows = int(os.environ.get("SIMPLY_B200_GATED_TC_MIN_ROWS", "129"))
    self.gated_tc_blocks = 0  # 0: one block per SM (tests: fewer, so that blocks walk many tiles)
    # Blocks work in pairs (tcgen05 cta_group::2, tiles of 256 tokens); False: each alone on tiles
    # of 128 (tests).  Measured at the Gemma 2 shapes: in short bursts single blocks are ahead on
    # the largest products (by 3 to 5 %), but whenever the GPU runs long enough for the power limit
    # to set the clocks (a prefill step of the 27B shape is 90 ms) pairs, which move a third less
    # data, are ahead at every size (by 2 to 4 %).
    self.gated_tc_pairs = True
    self.mid_rows = {"qkv": 32, "gated": 32, "plain": 32, "head": 32}
    env = os.environ.get("SIMPLY_B200_SERVING_BATCH_PRODUCT")  # experiments: "qkv:128,gated:32,plain:0,head:128"
    if env:
      for item in env.split(","):
        name, _, rows = item.partition(":")
        self.mid_rows[name] = int(rows or 128)
    self.mid_split = 0
    self.mid_stages = 0  # 0: the launch chooses the depth of the ring of stages; 8 deep, 4 shallow (tests)
    # The true 32-bit path must not be routed through a reduced-precision matrix mode.
    torch.backends.cuda.matmul.allow_tf32 = False
    self.launches = 0

  # ---- plumbing -------------------------------------------------------------
  def _declare(self) -> None:
    c_int, c_float, c_void, c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong
    protos = {
        "sb_embed": [c_void, c_int, c_void, c_float, c_void, c_int, c_int, c_int, c_void, c_void],
        "sb_residual_norm": [c_void, c_void, c_int, c_void, c_int, c_float, c_int, c_void, c_int, c_float,
                             c_int, c_void, c_void, c_int, c_int, c_int, c_void, c_void],
        "sb_rms_norm": [c_void, c_int, c_void, c_int, c_float, c_int, c_void, c_int, c_int, c_int, c_void],
        "sb_gather_rows": [c_void, c_int, c_void, c_void, c_int, c_int, c_int, c_void, c_void],
        "sb_add_to_residual": [c_void, c_void, c_int, c_ll, c_void],
        "sb_cast": [c_void, c_int, c_void, c_int, c_ll, c_void],
        "sb_rotation_tables": [c_void, c_void, c_float, c_void, c_void, c_int, c_int, c_void],
        "sb_rope_cache_write": [c_void, c_int, c_void, c_void, c_float, c_void, c_void, c_void, c_int, c_void,
                                c_void, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void, c_void],
        "sb_gated_activation": [c_void, c_int, c_void, c_int, c_int, c_int, c_void],
        "sb_soft_cap": [c_void, c_float, c_ll, c_void],
        "sb_gemm_f32_nt": [c_void, c_void, c_void, c_int, c_int, c_int, c_float, c_void],
        "sb_gemm_skinny_bf16": [c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void],
        "sb_gemm_stream_tc": [c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                              c_void, c_void],
        "sb_gemm_gated_tc": [c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_int, c_int, c_void, c_void],
        "sb_qkv_rope_stream_tc": [c_void, c_void, c_int, c_int, c_void, c_void, c_float, c_void, c_void, c_void, c_int,
                                  c_void, c_void, c_int, c_int, c_int, c_int, c_int, c_void, c_int, c_int, c_void],
        "sb_qkv_rope_skinny": [c_void, c_void, c_int, c_int, c_void, c_void, c_float, c_void, c_void, c_void, c_int,
                               c_void, c_void, c_int, c_int, c_int, c_int, c_int, c_void, c_int, c_void],
        "sb_paged_attention_generic": [c_void, c_int, c_void, c_void, c_int, c_void, c_void, c_void, c_int,
                                       c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void, c_void],
        "sb_sample": [c_void, c_void, c_void, c_int, c_int, c_void, c_void],
        "sb_sample_logprobs": [c_void, c_void, c_void, c_void, c_void, c_int, c_int, c_void, c_void],
        "sb_decode_advance": [c_void, c_void, c_void, c_void, c_void, c_void, c_void, c_int, c_void],
        "sb_keep_logits": [c_void, c_void, c_void, c_ll, c_void],
    }
    for name, argtypes in protos.items():
      fn = getattr(self.lib, name)
      fn.argtypes = argtypes
      fn.restype = c_int
    self.lib.sb_gemm_library_bf16.argtypes = [c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_void, c_ll, c_void]
    self.lib.sb_gemm_library_bf16.restype = c_int
    self.lib.sb_graph_burst.argtypes = [c_void, c_void, c_void, c_ll, c_int, c_void, c_void, c_ll, c_void]
    self.lib.sb_graph_burst.restype = c_int
    self.lib.sb_stream_wait.argtypes = [c_void]
    self.lib.sb_stream_wait.restype = c_int
    self.lib.sb_sample_slices.argtypes = [c_int, c_int]
    self.lib.sb_sample_slices.restype = c_int

  def _stream(self):
    if self._step_stream is not None:
      return self._step_stream
    return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

  def hold_stream(self):
    """Context in which every launch goes to the stream that is current now, looked up once
    instead of once per launch (an engine step is a few hundred launches)."""
    return _HeldStream(self)

  def _library_product(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """out = x . w^T through the matrix-product library with a kept algorithm; False when it
    has none for this shape."""
    stream = self._stream()
    workspace = self._library_workspaces.get(stream.value)
    if workspace is None:  # one per stream: products on different streams may run together
      workspace = self._library_workspaces[stream.value] = torch.empty(32 << 20, dtype=torch.uint8, device=self.device)
    m, k = x.shape
    rc = self.lib.sb_gemm_library_bf16(_ptr(x), _ptr(w), _ptr(out), m, w.shape[0], k, int(out.dtype == torch.float32),
                                       _ptr(workspace), workspace.numel(), stream)
    if rc > 0:
      raise KernelError(f"sb_gemm_library_bf16: cuBLAS status {rc}")
    self.launches += rc == 0
    return rc == 0

  def _call(self, name: str, *args) -> int:
    rc = getattr(self.lib, name)(*args, self._stream())
    self.launches += rc != -9  # -9: the kernel does not take the shape and launched nothing
    if rc != 0 and rc != -9:
      why = _STATUS.get(rc, f"CUDA error {rc}" if rc > 0 else f"status {rc}")
      raise KernelError(f"{name}: {why}")
    return rc

  def _new(self, *shape, dtype=None) -> torch.Tensor:
    return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

  def check_errors(self) -> None:
    """Reads the device error word (synchronises); raises if a kernel refused an access."""
    word = int(self.err.item())
    if word:
      self.err.zero_()
      reasons = [msg for bit, msg in _ERRORS.items() if word & bit]
      raise KernelError("a kernel skipped an invalid access: " + "; ".join(reasons))

  # ---- checks ---------------------------------------------------------------
  def check_attention(self, head_dim: int, num_heads: int, num_kv_heads: int) -> None:
    """Refuses shapes no kernel takes; compiles the tensor-core kernels of this head size."""
    if head_dim <= 0 or head_dim % 2 or head_dim > 512:
      raise KernelError(f"attention kernels take even head sizes up to 512, got {head_dim}")
    if num_heads % num_kv_heads:
      raise KernelError(f"{num_heads} query heads are no multiple of {num_kv_heads} key/value heads")
    if self._uses_tensor_core_attention(head_dim, num_heads // num_kv_heads):
      self._attention_lib(head_dim)

  def _uses_tensor_core_attention(self, head_dim: int, group: int) -> bool:
    return (self.dtype == torch.bfloat16 and self.tensor_core_attention and head_dim % 16 == 0
            and head_dim <= 256 and group <= 64)  # a group must fit a 64-row tile

  def _attention_lib(self, head_dim: int):
    fns = self._attn_fns.get(head_dim)
    if fns is None:
      lib = build.load_attention(head_dim)
      c_int, c_float, c_void = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
      prefill = getattr(lib, f"sb_attn_prefill_hd{head_dim}")
      prefill.argtypes = [c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_int, c_int, c_int, c_int,
                          c_float, c_int, c_void, c_int, c_int, c_int, c_void, c_void]
      prefill.restype = c_int
      decode = getattr(lib, f"sb_attn_decode_hd{head_dim}")
      decode.argtypes = [c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_void, c_int, c_int, c_int,
                         c_int, c_int, c_float, c_int, c_void, c_int, c_int, c_void, c_void, c_void, c_int,
                         c_void, c_void, c_int, c_void, c_int, c_void, c_void]
      decode.restype = c_int
      make_map = getattr(lib, f"sb_attn_tensor_map_hd{head_dim}")
      make_map.argtypes = [c_void, c_void, ctypes.c_longlong, c_int]
      make_map.restype = c_int
      prefill_tc = None
      if head_dim % 64 == 0:
        prefill_tc = getattr(lib, f"sb_attn_prefill_tc_hd{head_dim}")
        prefill_tc.argtypes = [c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_int, c_int, c_int, c_int,
                               c_int, c_float, c_int, c_void, c_int, c_void, c_void]
        prefill_tc.restype = c_int
      prefill_pair = None
      if head_dim in (128, 256):
        prefill_pair = getattr(lib, f"sb_attn_prefill_pair_hd{head_dim}")
        prefill_pair.argtypes = [c_void, c_void, c_void, c_int, c_void, c_void, c_void, c_int, c_int, c_int, c_int,
                                 c_int, c_float, c_int, c_void, c_int, c_void, c_void]
        prefill_pair.restype = c_int
      resident = getattr(lib, f"sb_attn_decode_resident_hd{head_dim}")
      resident.argtypes, resident.restype = [c_int], c_int
      slots = resident(1)
      if slots <= 0:
        raise KernelError(f"sb_attn_decode_resident: {_STATUS.get(slots, slots)}")
      self._decode_slots[head_dim] = slots
      fns = self._attn_fns[head_dim] = (prefill, decode, make_map, prefill_tc, prefill_pair)
    return fns

  def decode_chunk_for(self, kv_lo: Sequence[int], kv_hi: Sequence[int], num_kv_heads: int, head_dim: int) -> int:
    """Chunk length of split-key attention for sequences that see the keys [kv_lo, kv_hi).

    A work item is one chunk of one (sequence, kv head); the kernel's persistent grid draws items
    from a counter.  With `slots` resident blocks the launch lasts about
    ceil(items / slots) * (chunk + fixed cost of an item), so the chunk is the multiple of 64 that
    makes this smallest: the items then fill the grid in whole rounds instead of leaving most
    blocks idle in the last one.
    """
    if self.decode_chunk:
      return self.decode_chunk
    self._attention_lib(head_dim)
    slots = self._decode_slots[head_dim]
    lo, hi = np.asarray(kv_lo, dtype=np.int64), np.asarray(kv_hi, dtype=np.int64)
    # (From 128 keys: with 64 a lone sequence's window layers were 13 % slower than with 128,
    # although their items fit the grid either way: twice the items and twice the chunks to merge.)
    best, best_cost = 128, None
    for chunk in range(128, 2048 + 1, 64):
      items = int(((hi - 1) // chunk - lo // chunk + 1).sum()) * num_kv_heads
      cost = -(-items // slots) * (chunk + self.DECODE_ITEM_COST)
      if best_cost is None or cost <= best_cost:
        best, best_cost = chunk, cost
    return best

  # Fixed cost of a split-key work item (pipeline fill, partial result, its share of the merge),
  # in keys: about 2 microseconds of a block's share of the memory bandwidth.
  DECODE_ITEM_COST = 48

  @staticmethod
  def decode_chunk_range(q_start: np.ndarray, steps: int, window: int | None, chunk: int) -> tuple[np.ndarray, np.ndarray]:
    """First and last chunk index per sequence that a decode burst of `steps` steps touches: from
    the lowest key visible at the first step to the highest at the last."""
    qs = np.asarray(q_start, dtype=np.int64)
    lo = np.maximum(qs - window + 1, 0) // 64 * 64 if window else np.zeros_like(qs)
    return lo // chunk, (qs + steps - 1) // chunk

  @staticmethod
  def static_decode_plan(q_start: np.ndarray, steps: int, window: int | None, chunk: int,
                         items_per_seq: int) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Work list of the split-key kernel for a decode burst replayed from a CUDA graph.

    Every sequence gets exactly `items_per_seq` items, so the launch has a fixed size:
    the chunks that hold keys between the lowest key visible at the first step and the
    highest at the last step, then fillers (sequence -1).  A chunk that holds nothing
    visible at some step of the burst yields an empty partial result there.
    Returns (items [B * items_per_seq, 2], split_start [B], split_count [B]).
    """
    b = len(q_start)
    items = np.full((b, items_per_seq, 2), -1, dtype=np.int32)
    count = np.zeros(b, dtype=np.int32)
    firsts, lasts = CudaOps.decode_chunk_range(q_start, steps, window, chunk)
    for i, (first, last) in enumerate(zip(firsts.tolist(), lasts.tolist())):
      n = last - first + 1
      if n > items_per_seq:
        raise KernelError(f"decode burst needs {n} chunks per sequence, the graph holds {items_per_seq}")
      items[i, :n, 0] = i
      items[i, :n, 1] = np.arange(first, last + 1)
      count[i] = n
    start = (np.arange(b) * items_per_seq).astype(np.int32)
    return items.reshape(-1, 2), start, count

  def _tensor_map(self, storage: torch.Tensor, head_dim: int, page_size: int):
    """TMA descriptor of a cache storage (made once per storage), or None where TMA cannot be used."""
    if head_dim % 64 or page_size & (page_size - 1):
      return None
    # The descriptor holds the storage's address and its number of rows (rows beyond read as
    # zeros): another storage that the allocator puts at the same address must not find it.
    key = (storage.data_ptr(), storage.numel(), head_dim, page_size)
    buf = self._tensor_maps.get(key)
    if buf is None:
      make_map = self._attention_lib(head_dim)[2]
      buf = ctypes.create_string_buffer(128 + 64)
      aligned = (ctypes.addressof(buf) + 63) & ~63
      tile_keys = 32 if head_dim > 128 else 64
      rc = make_map(ctypes.c_void_p(aligned), _ptr(storage), storage.numel() // head_dim, min(page_size, tile_keys))
      buf = (buf, aligned if rc == 0 else None)
      self._tensor_maps[key] = buf
    return ctypes.c_void_p(buf[1]) if buf[1] is not None else None

  def _prefill_uses_tcgen05(self, head_dim: int, group: int, page_size: int) -> bool:
    return (self.prefill_tcgen05 and head_dim % 64 == 0 and 128 % group == 0
            and page_size & (page_size - 1) == 0)

  def _prefill_uses_pairs(self, head_dim: int, group: int, page_size: int) -> bool:
    """The tcgen05 prefill kernel by pairs of blocks (csrc/attention_tc_pair.cu)."""
    return (self.prefill_pairs and self._prefill_uses_tcgen05(head_dim, group, page_size)
            and head_dim in (128, 256) and page_size >= 64)

  def _prefill_rows(self, head_dim: int, group: int, page_size: int) -> int:
    """Query rows of a prefill work item: 256 for a pair of blocks, 128 for the tcgen05 kernel, else the mma.sync tile."""
    if self._prefill_uses_pairs(head_dim, group, page_size):
      return 256
    if self._prefill_uses_tcgen05(head_dim, group, page_size):
      return 128
    return self.prefill_rows or 64

  def _plan_key(self, window: int | None, group: int, num_kv_heads: int, head_dim: int, page_size: int) -> tuple:
    """Where a step keeps the work lists of one kind of attention layer in `ctx.memo`.  Layers
    share lists only if everything the lists are cut for agrees: the window, the group, the
    number of kv heads and the head size (they set the chunk length) and the rows of a prefill tile."""
    return ("attention_plan", window, group, num_kv_heads, head_dim, self._prefill_rows(head_dim, group, page_size))

  def attention_graph_plan(self, *, window: int | None, num_heads: int, num_kv_heads: int, head_dim: int,
                           batch: int, bucket: int, max_burst: int, page_size: int):
    """The static work list a decode graph needs for one kind of attention layer, or None when
    the kernel that serves it reads no list (the general kernel)."""
    group = num_heads // num_kv_heads
    if not self._uses_tensor_core_attention(head_dim, group):
      return None
    return AttentionGraphPlan(self, window, group, num_kv_heads, head_dim, batch, bucket, max_burst, page_size)

  def _attention_plan(self, ctx: Any, window: int | None, group: int, force_rows: int = 0,
                      num_kv_heads: int = 1, head_dim: int = 0) -> dict:
    """Work lists of the two tensor-core kernels for this step, per kind of layer (`_plan_key`).

    Sequences with at most 16 query rows per kv head (one or a few new tokens) go to the
    split-key kernel: their keys are cut into chunks at multiples of `chunk` of the
    absolute position, one work item per chunk.  The others are cut into tiles of
    64 // group or 128 // group tokens for the prefill kernel, heaviest tile first.
    """
    key = self._plan_key(window, group, num_kv_heads, head_dim, ctx.page_size)
    plan = ctx.memo.get(key)
    if plan is not None:
      return plan
    cu_q, q_start = ctx.host["cu_q"], ctx.host["q_start"].astype(np.int64)
    q_len = np.diff(cu_q).astype(np.int64)
    small = q_len * group <= 16
    # Tiles of 64 query rows (finer grains balance better over the SMs than tiles of 128).
    rows_per_tile = force_rows or self.prefill_rows or 64
    tokens_per_tile = rows_per_tile // group
    num_seqs = len(q_len)
    pre = []
    for b in np.nonzero(~small)[0]:
      for i0 in range(0, int(q_len[b]), tokens_per_tile):
        last = int(q_start[b]) + min(i0 + tokens_per_tile, int(q_len[b]))
        first = max(int(q_start[b]) + i0 - window + 1, 0) if window else 0
        pre.append((last - first, int(b), i0))
    pre.sort(key=lambda x: -x[0])
    if force_rows in (128, 256):
      # The tcgen05 kernels' blocks, one per (tile of queries, kv head), longest walk first over all
      # heads: the GPU holds 74 pairs (or 148 single blocks) at once and gives the next one in the list to the SMs that
      # are free first, so this order fills them evenly (listed head by head, 128 blocks of a
      # 4,096-token prompt ended as late as 53 tiles' time where 37 are enough).
      prefill_items = np.array([(b, i0, m) for _, b, i0 in pre for m in range(num_kv_heads)],
                               dtype=np.int32).reshape(-1, 3)
    else:
      prefill_items = np.array([(b, i0) for _, b, i0 in pre], dtype=np.int32).reshape(-1, 2)
    kv_hi = q_start + q_len
    kv_lo = np.maximum(q_start - window + 1, 0) if window else np.zeros_like(q_start)
    kv_lo = kv_lo // 64 * 64
    dec = np.nonzero(small)[0]
    chunk = 64
    if len(dec):
      chunk = self.decode_chunk_for(kv_lo[dec], kv_hi[dec], num_kv_heads, head_dim)
    split_start = np.zeros(num_seqs, dtype=np.int32)
    split_count = np.zeros(num_seqs, dtype=np.int32)
    dec_items = []
    for b in dec:
      first, last = int(kv_lo[b]) // chunk, (int(kv_hi[b]) - 1) // chunk
      split_start[b] = len(dec_items)
      split_count[b] = last - first + 1
      dec_items += [(int(b), c) for c in range(first, last + 1)]
    decode_items = np.array(dec_items, dtype=np.int32).reshape(-1, 2)
    flat = np.concatenate([prefill_items.reshape(-1), decode_items.reshape(-1), split_start, split_count])
    dev = torch.from_numpy(flat).to(self.device, non_blocking=True)
    n_pre, n_dec = prefill_items.size, decode_items.size
    plan = dict(
        num_prefill=len(prefill_items), num_decode=len(decode_items), chunk=chunk, rows_per_tile=rows_per_tile,
        rows_max=int((q_len[dec] * group).max()) if len(dec) else 0,
        prefill_items=dev[:n_pre], decode_items=dev[n_pre:n_pre + n_dec],
        split_start=dev[n_pre + n_dec:n_pre + n_dec + num_seqs], split_count=dev[n_pre + n_dec + num_seqs:])
    ctx.memo[key] = plan
    return plan

  # ---- dense ----------------------------------------------------------------
  def embed(self, table: torch.Tensor, ids: torch.Tensor, scale: float) -> torch.Tensor:
    if table.dtype == torch.bfloat16:
      # The reference rounds the constant to the activation dtype (simply/utils/module.py:477-481).
      rounded = self._rounded_scales.get(scale)
      if rounded is None:
        rounded = self._rounded_scales[scale] = float(torch.tensor(scale, dtype=torch.float32).to(torch.bfloat16))
      scale = rounded
    out = self._new(ids.numel(), table.shape[1], dtype=torch.float32)
    self._call("sb_embed", _ptr(table), _code(table), _ptr(ids), float(scale), _ptr(out), ids.numel(),
               table.shape[1], table.shape[0], _ptr(self.err))
    return out

  def cast(self, x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if x.dtype == dtype:
      return x
    out = self._new(*x.shape, dtype=dtype)
    self._call("sb_cast", _ptr(x), _code(x), _ptr(out), _code(out), x.numel())
    return out

  def _mid_product(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, cap: float = 0.0,
                   activation: int = 0, split: int | None = None) -> bool:
    """The weight-streaming product for a serving batch (17 to 128 tokens); False when it does
    not take the shape."""
    m, k = x.shape
    n = w.shape[0]
    split = self.mid_split if split is None else split
    return self._call("sb_gemm_stream_tc", _ptr(x), _ptr(w), _ptr(out), m, n, k, epilogue, float(cap), activation,
                      split, self.mid_stages, _ptr(self.err)) == 0

  def linear(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [M, K] . w[N, K]^T -> [M, N] in the activation dtype."""
    m, k = x.shape
    n = w.shape[0]
    if w.dtype == torch.float32:
      # Float32 weights (the 32-bit path, or a tensor stored in 32 bits): true float32 product.
      xf = self.cast(x, torch.float32)
      out = self._new(m, n, dtype=torch.float32)
      self._call("sb_gemm_f32_nt", _ptr(xf), _ptr(w), _ptr(out), m, n, k, 0.0)
      return self.cast(out, self.dtype)
    x = self.cast(x, torch.bfloat16)
    if m <= self.skinny_max_rows:
      out = self._new(m, n, dtype=torch.bfloat16)
      if self._call("sb_gemm_skinny_bf16", _ptr(x), _ptr(w), _ptr(out), m, n, k, 0, 0.0, 0, self.skinny_warps) == 0:
        return out
    elif m <= self.mid_rows["plain"] and self.mid_rows_kernel and x.is_contiguous() and w.is_contiguous():
      out = self._new(m, n, dtype=torch.bfloat16)
      if self._mid_product(x, w, out, 0):
        return out
    if self.direct_library_products and x.is_contiguous() and w.is_contiguous():
      out = self._new(m, n, dtype=torch.bfloat16)
      if self._library_product(x, w, out):
        return out
    return torch.mm(x, w.t())

  def gated_linear(self, x: torch.Tensor, w_gate_up: torch.Tensor, activation: int) -> torch.Tensor:
    """act(x . w_gate^T) * (x . w_up^T) with w_gate_up = [gate rows; up rows]: [M, N/2]."""
    m, k = x.shape
    n = w_gate_up.shape[0]
    if w_gate_up.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and m <= self.skinny_max_rows:
      out = self._new(m, n // 2, dtype=torch.bfloat16)
      if self._call("sb_gemm_skinny_bf16", _ptr(x), _ptr(w_gate_up), _ptr(out), m, n, k, 2, 0.0,
                    activation, self.skinny_warps) == 0:
        return out
    if (w_gate_up.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and self.mid_rows_kernel
        and self.skinny_max_rows < m <= self.mid_rows["gated"] and x.is_contiguous() and w_gate_up.is_contiguous()):
      out = self._new(m, n // 2, dtype=torch.bfloat16)
      if self._mid_product(x, w_gate_up, out, 2, activation=activation):
        return out
    if (w_gate_up.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and m >= self.gated_tc_min_rows > 0
        and x.is_contiguous() and w_gate_up.is_contiguous()):
      out = self._new(m, n // 2, dtype=torch.bfloat16)
      if self._call("sb_gemm_gated_tc", _ptr(x), _ptr(w_gate_up), _ptr(out), m, n // 2, k, activation,
                    self.gated_tc_blocks, int(self.gated_tc_pairs), _ptr(self.err)) == 0:
        return out
    return self.gated_activation(self.linear(x, w_gate_up), activation)

  def lm_head(self, x: torch.Tensor, table: torch.Tensor, cap: float) -> torch.Tensor:
    """float32 logits [R, vocab] = softcap(x . table^T)."""
    r, k = x.shape
    v = table.shape[0]
    out = self._new(r, v, dtype=torch.float32)
    if table.dtype == torch.float32:
      xf = self.cast(x, torch.float32)
      self._call("sb_gemm_f32_nt", _ptr(xf), _ptr(table), _ptr(out), r, v, k, float(cap))
      return out
    x = self.cast(x, torch.bfloat16)
    chunk = 32
    if chunk < r <= self.mid_rows["head"] and self.mid_rows_kernel and k % 8 == 0 and x.is_contiguous():
      # 33 to 128 rows: one pass over the table instead of several
      if self._mid_product(x, table, out, 1, cap=cap, split=1):
        return out
    if r > chunk and k % 8 == 0:
      if self.direct_library_products and x.is_contiguous() and self._library_product(x, table, out):
        self._call("sb_soft_cap", _ptr(out), float(cap), out.numel())
        return out
      try:
        torch.mm(x, table.t(), out_dtype=torch.float32, out=out)
        self._call("sb_soft_cap", _ptr(out), float(cap), out.numel())
        return out
      except (TypeError, RuntimeError):
        pass
    if k % 8:
      raise KernelError(f"the output layer's width {k} must be a multiple of 8 in bfloat16")
    for r0 in range(0, r, chunk):
      rows = min(chunk, r - r0)
      self._call("sb_gemm_skinny_bf16", _ptr(x[r0:]), _ptr(table), _ptr(out[r0:]), rows, v, k, 1,
                 float(cap), 0, self.skinny_warps)
    return out

  def gated_activation(self, gate_up: torch.Tensor, activation: int) -> torch.Tensor:
    t, two_f = gate_up.shape
    out = self._new(t, two_f // 2, dtype=gate_up.dtype)
    self._call("sb_gated_activation", _ptr(gate_up), _code(gate_up), _ptr(out), t, two_f // 2, activation)
    return out

  # ---- norms ----------------------------------------------------------------
  def rms_norm(self, x: torch.Tensor, w: torch.Tensor, eps: float, plus_one: bool) -> torch.Tensor:
    out = self._new(*x.shape)
    self._call("sb_rms_norm", _ptr(x), _code(x), _ptr(w), int(w.dtype == torch.float32), float(eps),
               int(plus_one), _ptr(out), _code(out), x.shape[0], x.shape[1])
    return out

  def residual_norm(self, h: torch.Tensor, branch: torch.Tensor | None, post: Any, pre: Any,
                    rows: torch.Tensor | None) -> torch.Tensor | None:
    """h += norm_post(branch); returns norm_pre(h) in the activation dtype (see csrc/elementwise.cu)."""
    width = h.shape[1]
    num_rows = h.shape[0] if rows is None else rows.numel()
    y = self._new(num_rows, width) if pre is not None else None
    if branch is None and pre is None:
      return None
    if branch is not None and branch.dtype != self.dtype:
      branch = self.cast(branch, self.dtype)
    wp, wq = (post.weight if post is not None else None), (pre.weight if pre is not None else None)
    self._call(
        "sb_residual_norm", _ptr(h), _ptr(branch), _BF16 if self.dtype == torch.bfloat16 else _F32,
        _ptr(wp), int(wp is not None and wp.dtype == torch.float32),
        float(post.eps) if post is not None else 0.0, int(post.plus_one) if post is not None else 0,
        _ptr(wq), int(wq is not None and wq.dtype == torch.float32),
        float(pre.eps) if pre is not None else 0.0, int(pre.plus_one) if pre is not None else 0,
        _ptr(rows), _ptr(y), num_rows, width, h.shape[0], _ptr(self.err))
    return y

  def gather_rows(self, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    out = self._new(rows.numel(), x.shape[1], dtype=x.dtype)
    self._call("sb_gather_rows", _ptr(x), _code(x), _ptr(rows), _ptr(out), rows.numel(), x.shape[1],
               x.shape[0], _ptr(self.err))
    return out

  def add_to_residual(self, h: torch.Tensor, x: torch.Tensor) -> None:
    self._call("sb_add_to_residual", _ptr(h), _ptr(x), _code(x), h.numel())

  # ---- positions ------------------------------------------------------------
  def rotation_tables(self, positions: torch.Tensor, timescale: torch.Tensor, scale_factor: float):
    t, half = positions.numel(), timescale.numel()
    cos = self._new(t, half, dtype=torch.float32)
    sin = self._new(t, half, dtype=torch.float32)
    self._call("sb_rotation_tables", _ptr(positions), _ptr(timescale), float(scale_factor), _ptr(cos),
               _ptr(sin), t, half)
    return cos, sin

  def rope_and_cache_write(self, qkv: torch.Tensor, tables, q_scale: float, num_heads: int,
                           num_kv_heads: int, head_dim: int, storage: torch.Tensor | None,
                           block_table: torch.Tensor, ctx: Any) -> torch.Tensor:
    t = qkv.shape[0]
    q = self._new(t, num_heads, head_dim, dtype=qkv.dtype)
    cos, sin = tables if tables is not None else (None, None)
    if storage is not None and storage.dtype != qkv.dtype:
      raise KernelError("cache and activations must share one dtype")
    self._call("sb_rope_cache_write", _ptr(qkv), _code(qkv), _ptr(cos), _ptr(sin), float(q_scale), _ptr(q),
               _ptr(storage), _ptr(block_table), block_table.shape[1], _ptr(ctx.token_seq),
               _ptr(ctx.positions), t, num_heads, num_kv_heads, head_dim, ctx.page_size,
               storage.shape[0] if storage is not None else 0, int(storage is not None), _ptr(self.err))
    return q

  def project_rotate_store(self, x: torch.Tensor, w_qkv: torch.Tensor, tables, q_scale: float, num_heads: int,
                           num_kv_heads: int, head_dim: int, storage: torch.Tensor | None,
                           block_table: torch.Tensor, ctx: Any) -> torch.Tensor:
    """The fused q, k, v projection, then rotation, query scale and the stores: queries
    [T, num_heads, head_dim] are returned, keys and values go into the pages of `storage`.

    Steps of a few tokens do it in one kernel (the product's epilogue rotates and stores);
    larger ones as a product followed by `rope_and_cache_write`.
    """
    t, k = x.shape
    if (self.fused_qkv_rope and self.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16
        and t <= self.skinny_max_rows and t <= 16 and head_dim % 32 == 0 and k % 8 == 0):
      x = self.cast(x, torch.bfloat16)
      q = self._new(t, num_heads, head_dim, dtype=torch.bfloat16)
      cos, sin = tables if tables is not None else (None, None)
      if storage is not None and storage.dtype != torch.bfloat16:
        raise KernelError("cache and activations must share one dtype")
      rc = self._call("sb_qkv_rope_skinny", _ptr(x), _ptr(w_qkv), t, k, _ptr(cos), _ptr(sin), float(q_scale),
                      _ptr(q), _ptr(storage), _ptr(block_table), block_table.shape[1], _ptr(ctx.token_seq),
                      _ptr(ctx.positions), num_heads, num_kv_heads, head_dim, ctx.page_size,
                      storage.shape[0] if storage is not None else 0, _ptr(self.err), self.skinny_warps)
      if rc == 0:
        return q
    if (self.fused_qkv_rope and self.mid_rows_kernel and self.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16
        and self.skinny_max_rows < t <= self.mid_rows["qkv"] and head_dim % 128 == 0 and k % 8 == 0):
      x = self.cast(x, torch.bfloat16)
      q = self._new(t, num_heads, head_dim, dtype=torch.bfloat16)
      cos, sin = tables if tables is not None else (None, None)
      if storage is not None and storage.dtype != torch.bfloat16:
        raise KernelError("cache and activations must share one dtype")
      args = (_ptr(x), _ptr(w_qkv), t, k, _ptr(cos), _ptr(sin), float(q_scale),
              _ptr(q), _ptr(storage), _ptr(block_table), block_table.shape[1], _ptr(ctx.token_seq),
              _ptr(ctx.positions), num_heads, num_kv_heads, head_dim, ctx.page_size,
              storage.shape[0] if storage is not None else 0, _ptr(self.err), self.mid_split)
      rc = self._call("sb_qkv_rope_stream_tc", *args, self.mid_stages)
      if rc == 0:
        return q
    qkv = self.linear(x, w_qkv)
    return self.rope_and_cache_write(qkv, tables, q_scale, num_heads, num_kv_heads, head_dim, storage,
                                     block_table, ctx)

  # ---- attention ------------------------------------------------------------
  def paged_attention(self, q: torch.Tensor, storage: torch.Tensor, block_table: torch.Tensor, ctx: Any, *,
                      num_heads: int, num_kv_heads: int, head_dim: int, logit_softcap: float,
                      window: int | None) -> torch.Tensor:
    t = q.shape[0]
    out = self._new(t, num_heads * head_dim, dtype=q.dtype)
    group = num_heads // num_kv_heads
    if q.dtype == torch.bfloat16 and self._uses_tensor_core_attention(head_dim, group):
      prefill, decode, _, prefill_tc, prefill_pair = self._attention_lib(head_dim)
      use_tc = prefill_tc is not None and self._prefill_uses_tcgen05(head_dim, group, ctx.page_size)
      use_pair = prefill_pair is not None and self._prefill_uses_pairs(head_dim, group, ctx.page_size)
      plan = self._attention_plan(ctx, window, group, 256 if use_pair else (128 if use_tc else 0), num_kv_heads, head_dim)
      common = (_ptr(q), _ptr(storage), _ptr(block_table), block_table.shape[1], _ptr(ctx.cu_q),
                _ptr(ctx.q_start))
      sizes = (num_heads, num_kv_heads, ctx.page_size, storage.shape[0], float(logit_softcap), int(window or 0))
      if plan["num_prefill"] and use_pair:
        rc = prefill_pair(*common, _ptr(out), t, *sizes, _ptr(plan["prefill_items"]), plan["num_prefill"],
                          _ptr(self.err), self._stream())
        self.launches += 1
        if rc:
          raise KernelError(f"sb_attn_prefill_pair: {_STATUS.get(rc, rc)}")
      elif plan["num_prefill"] and use_tc:
        rc = prefill_tc(*common, _ptr(out), t, *sizes, _ptr(plan["prefill_items"]), plan["num_prefill"],
                        _ptr(self.err), self._stream())
        self.launches += 1
        if rc:
          raise KernelError(f"sb_attn_prefill_tc: {_STATUS.get(rc, rc)}")
      elif plan["num_prefill"]:
        rc = prefill(*common, _ptr(out), *sizes, _ptr(plan["prefill_items"]), plan["num_prefill"],
                     plan["rows_per_tile"], int(self.prefill_single_key_group), _ptr(self.err), self._stream())
        self.launches += 1
        if rc:
          raise KernelError(f"sb_attn_prefill: {_STATUS.get(rc, rc)}")
      if plan["num_decode"]:
        n = plan["num_decode"] * num_kv_heads * plan["rows_max"]
        part_o = self._new(n * head_dim, dtype=torch.float32)
        part_ml = self._new(n * 2, dtype=torch.float32)
        rc = decode(*common, _ptr(ctx.token_seq), _ptr(out), t, *sizes, _ptr(plan["decode_items"]),
                    plan["num_decode"], plan["chunk"], _ptr(part_o), _ptr(part_ml), _ptr(self._attn_counter),
                    plan["rows_max"],
                    _ptr(plan["split_start"]), _ptr(plan["split_count"]), self.decode_variant,
                    self._tensor_map(storage, head_dim, ctx.page_size),
                    int(getattr(ctx, "older_keys_settled", False)), _ptr(self.err), self._stream())
        self.launches += 2
        if rc:
          raise KernelError(f"sb_attn_decode: {_STATUS.get(rc, rc)}")
      return out
    self._call("sb_paged_attention_generic", _ptr(q), _code(q), _ptr(storage), _ptr(block_table),
               block_table.shape[1], _ptr(ctx.token_seq), _ptr(ctx.positions), _ptr(out), t, num_heads,
               num_kv_heads, head_dim, ctx.page_size, storage.shape[0], float(logit_softcap),
               int(window or 0), _ptr(self.err))
    return out

  # ---- sampling -------------------------------------------------------------
  def sample(self, logits: torch.Tensor, temperature, top_k, top_p, seed, position, logprobs: bool = False):
    """One token per row of float32 logits; the other arguments are host sequences.  With
    `logprobs` also the float32 log-probability of each token under the distribution it was
    drawn from (0 for greedy rows): (tokens, logprobs)."""
    params = self.pack_sample_params(temperature, top_k, top_p, seed, position)
    dev_params = torch.from_numpy(params).to(self.device, non_blocking=True)
    if not logprobs:
      return self.sample_device(logits, dev_params)
    lp = self._new(logits.shape[0], dtype=torch.float32)
    return self.sample_device(logits, dev_params, logprobs_out=lp), lp

  @staticmethod
  def pack_sample_params(temperature, top_k, top_p, seed, position) -> np.ndarray:
    """The [R, 6] int32 words the sampling kernel reads (see csrc/sampling.cu)."""
    r = len(temperature)
    params = np.zeros((r, 6), dtype=np.int32)
    params[:, 0] = np.asarray(temperature, dtype=np.float32).view(np.int32)
    params[:, 1] = np.asarray(top_k, dtype=np.int32)
    params[:, 2] = np.asarray(top_p, dtype=np.float32).view(np.int32)
    seeds = np.asarray([int(s) & 0xFFFFFFFFFFFFFFFF for s in seed], dtype=np.uint64)
    params[:, 3] = (seeds & np.uint64(0xFFFFFFFF)).astype(np.uint32).view(np.int32)
    params[:, 4] = (seeds >> np.uint64(32)).astype(np.uint32).view(np.int32)
    params[:, 5] = np.asarray(position, dtype=np.int32)
    return params

  def sample_device(self, logits: torch.Tensor, dev_params: torch.Tensor, out: torch.Tensor | None = None,
                    logprobs_out: torch.Tensor | None = None, step_counter: torch.Tensor | None = None) -> torch.Tensor:
    """Sampling with the parameter words already on the device.  `logprobs_out` (float32 [R], or
    [steps, R] indexed by the device-side `step_counter`) receives the tokens' log-probabilities."""
    r, vocab = logits.shape
    if out is None:
      out = self._new(r, dtype=torch.int32)
    slices = self.lib.sb_sample_slices(r, vocab)
    scratch = self._new(r * (2 + 2 * slices), dtype=torch.int32)
    logits = logits.contiguous()
    self._call("sb_sample", _ptr(logits), _ptr(dev_params), _ptr(out), r, vocab, _ptr(scratch))
    self.launches += 2
    if logprobs_out is not None:
      self._call("sb_sample_logprobs", _ptr(logits), _ptr(dev_params), _ptr(out), _ptr(logprobs_out),
                 _ptr(step_counter), r, vocab, _ptr(scratch))
    return out

  def token_logprobs(self, logits: torch.Tensor, tokens: torch.Tensor, temperature: float, top_k: int,
                     top_p: float) -> torch.Tensor:
    """float32 [R]: the log-likelihood of tokens[r] under row r of `logits` with the sampling masks
    applied (simply/utils/sampling_lib.py:540-601): a greedy setting scores the argmax 0 and every
    other token -inf; otherwise the log-softmax of logits / temperature over the kept entries."""
    r, vocab = logits.shape
    logits = logits.contiguous()
    params = self.pack_sample_params([temperature] * r, [top_k] * r, [top_p] * r, [0] * r, [0] * r)
    dev_params = torch.from_numpy(params).to(self.device, non_blocking=True)
    slices = self.lib.sb_sample_slices(r, vocab)
    scratch = self._new(r * (2 + 2 * slices), dtype=torch.int32)
    drawn = self._new(r, dtype=torch.int32)
    # (the draw is not used, except for greedy rows, where it is the argmax; the call leaves the
    # rows' keep-thresholds in `scratch`)
    self._call("sb_sample", _ptr(logits), _ptr(dev_params), _ptr(drawn), r, vocab, _ptr(scratch))
    out = self._new(r, dtype=torch.float32)
    tokens = tokens.to(device=self.device, dtype=torch.int32).contiguous()
    self._call("sb_sample_logprobs", _ptr(logits), _ptr(dev_params), _ptr(tokens), _ptr(out), None, r, vocab,
               _ptr(scratch))
    if temperature == 0 or top_k == 1:
      out = torch.where(tokens == drawn, out, torch.full_like(out, float("-inf")))
    else:
      out = torch.where(out <= -3.0e38, torch.full_like(out, float("-inf")), out)  # a token the masks drop
    return out

  def keep_logits(self, logits: torch.Tensor, history: torch.Tensor, step_counter: torch.Tensor) -> None:
    """history[step_counter] = logits, without the host knowing the step (tests of graph replays)."""
    self._call("sb_keep_logits", _ptr(logits), _ptr(history), _ptr(step_counter), logits.numel())

  def decode_advance(self, sampled, token_ids, positions, q_start, sample_params, history, step_counter) -> None:
    self._call("sb_decode_advance", _ptr(sampled), _ptr(token_ids), _ptr(positions), _ptr(q_start),
               _ptr(sample_params), _ptr(history), _ptr(step_counter), sampled.numel())
