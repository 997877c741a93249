"""Loads a model's tensors by name from a safetensors folder, with one clear error.

The model says which tensors it needs (`TensorSpec`s: name, shape, kind); the
loader compares that list with what the files hold and reports *all* missing
tensors, unexpected tensors and wrong shapes in a single `WeightError`.  The
reference checks shapes one leaf at a time and only warns about missing leaves
(simply/utils/checkpoint_lib.py:754-758, :769-773); here nothing is loaded
unless the whole table matches.

Storage rule.  In float32 mode every floating tensor becomes float32.  In
bfloat16 mode a tensor stored in bfloat16 (or float16) is kept in bfloat16.  A
tensor stored in 32 bits follows its spec's `precision`: "activation" (operands
of matrix products and the embedding table) is narrowed to bfloat16, as the
reference narrows every wider float to the activation dtype on restore
(simply/serving/page_batcher.py:149-166, simply/utils/checkpoint_lib.py:658-670),
so that a folder published in float32 takes the memory and the kernels of the
bfloat16 path; "stored" (norm scales, and whatever a part declares so: router
weights, decay rates) stays in 32 bits.  `keep_float32=True` keeps every
32-bit tensor as stored.  Integer tables become int32.
"""

from __future__ import annotations

import dataclasses
import sys
from typing import Iterable

import torch

from simply_b200.weights import safetensors_io as st


@dataclasses.dataclass(frozen=True)
class TensorSpec:
  """A tensor the model needs.

  kind: "matrix" (weights of a linear map or an embedding table), "scale"
    (a norm's per-channel scale) or "table" (integers).  The kind decides how
    random-weights mode fills it; the loader only uses it for integer tables.
  optional: may be absent from the files (e.g. a duplicate of a tied table).
  precision: "activation" (narrowed to the activation dtype on load), "stored" (a tensor stored
    in 32 bits stays in 32 bits) or None: "stored" for scales, "activation" otherwise.
  """

  name: str
  shape: tuple[int, ...]
  kind: str = "matrix"
  optional: bool = False
  precision: str | None = None

  def keeps_stored_precision(self) -> bool:
    if self.precision is None:
      return self.kind == "scale"
    if self.precision not in ("activation", "stored"):
      raise ValueError(f"{self.name}: precision must be 'activation' or 'stored', got {self.precision!r}")
    return self.precision == "stored"


class WeightError(ValueError):
  """The files do not hold exactly the tensors the model needs."""

  def __init__(self, missing, unexpected, wrong_shape, wrong_kind=(), other=()):
    self.missing = list(missing)
    self.unexpected = list(unexpected)
    self.wrong_shape = list(wrong_shape)
    self.wrong_kind = list(wrong_kind)
    self.other = list(other)
    lines = ["model weights do not match the model:"]
    if self.missing:
      lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
    if self.unexpected:
      lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
    for name, want, got in self.wrong_shape:
      lines.append(f"  wrong shape: {name} is {list(got)} in the file, the model needs {list(want)}")
    for name, want, got in self.wrong_kind:
      lines.append(f"  wrong dtype class: {name} is stored as {got}, the model needs {want}")
    lines += [f"  {msg}" for msg in self.other]
    super().__init__("\n".join(lines))


def check(specs: Iterable[TensorSpec], entries: dict[str, st.TensorEntry]) -> None:
  """Raises WeightError unless `entries` holds exactly what `specs` lists."""
  specs = list(specs)
  by_name = {s.name: s for s in specs}
  missing = [s.name for s in specs if s.name not in entries and not s.optional]
  unexpected = sorted(n for n in entries if n not in by_name)
  wrong_shape, wrong_kind = [], []
  for s in specs:
    e = entries.get(s.name)
    if e is None:
      continue
    if tuple(e.shape) != tuple(s.shape):
      wrong_shape.append((s.name, tuple(s.shape), tuple(e.shape)))
    if (s.kind == "table") == e.is_float:
      wrong_kind.append((s.name, "integers" if s.kind == "table" else "floating point", e.dtype))
  if missing or unexpected or wrong_shape or wrong_kind:
    raise WeightError(missing, unexpected, wrong_shape, wrong_kind)


def target_dtype(entry: st.TensorEntry, activation_dtype: torch.dtype, spec: TensorSpec | None = None,
                 keep_float32: bool = False) -> torch.dtype:
  if not entry.is_float:
    return torch.int32
  if activation_dtype == torch.float32:
    return torch.float32
  if entry.is_32bit_float and (keep_float32 or spec is None or spec.keeps_stored_precision()):
    return torch.float32
  return torch.bfloat16


def load_tensors(
    model_dir: str,
    specs: Iterable[TensorSpec],
    activation_dtype: torch.dtype,
    device: torch.device | str,
    keep_float32: bool = False,
) -> dict[str, torch.Tensor]:
  """Checks the folder against `specs` and returns name -> tensor on `device`."""
  specs = list(specs)
  entries = st.index_files(st.model_files(model_dir))
  check(specs, entries)
  reader = st.TensorReader(entries)
  out: dict[str, torch.Tensor] = {}
  narrowed = 0
  try:
    for s in specs:
      if s.name not in entries:
        continue
      t = reader.read(s.name)
      dtype = target_dtype(entries[s.name], activation_dtype, s, keep_float32)
      narrowed += entries[s.name].is_32bit_float and dtype == torch.bfloat16
      out[s.name] = t.to(device=device, dtype=dtype)
  finally:
    reader.close()
  if narrowed:
    print(f"[simply_b200] {narrowed} tensor(s) stored in 32 bits were narrowed to bfloat16, the activation "
          "dtype (keep_float32_weights keeps them)", file=sys.stderr, flush=True)
  return out
