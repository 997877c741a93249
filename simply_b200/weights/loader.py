"""Loads a model's tensors by name from a safetensors folder, with one clear error.

The model says which tensors it needs (`TensorSpec`s: name, shape, kind); the
loader compares that list with what the files hold and reports *all* missing
tensors, unexpected tensors and wrong shapes in a single `WeightError`.  The
reference checks shapes one leaf at a time and only warns about missing leaves
(simply/utils/checkpoint_lib.py:754-758, :769-773); here nothing is loaded
unless the whole table matches.

Storage rule: floating tensors are kept in bfloat16 when the engine runs in
bfloat16, except that a tensor stored in 32 bits stays in 32 bits; in float32
mode every floating tensor becomes float32.  Integer tables become int32.
(The reference narrows wider floats to the activation dtype on restore,
simply/serving/page_batcher.py:149-166.)
"""

from __future__ import annotations

import dataclasses
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
  """

  name: str
  shape: tuple[int, ...]
  kind: str = "matrix"
  optional: bool = False


class WeightError(ValueError):
  """The files do not hold exactly the tensors the model needs."""

  def __init__(self, missing, unexpected, wrong_shape, wrong_kind=()):
    self.missing = list(missing)
    self.unexpected = list(unexpected)
    self.wrong_shape = list(wrong_shape)
    self.wrong_kind = list(wrong_kind)
    lines = ["model weights do not match the model:"]
    if self.missing:
      lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
    if self.unexpected:
      lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
    for name, want, got in self.wrong_shape:
      lines.append(f"  wrong shape: {name} is {list(got)} in the file, the model needs {list(want)}")
    for name, want, got in self.wrong_kind:
      lines.append(f"  wrong dtype class: {name} is stored as {got}, the model needs {want}")
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


def target_dtype(entry: st.TensorEntry, activation_dtype: torch.dtype) -> torch.dtype:
  if not entry.is_float:
    return torch.int32
  if activation_dtype == torch.float32 or entry.is_32bit_float:
    return torch.float32
  return torch.bfloat16


def load_tensors(
    model_dir: str,
    specs: Iterable[TensorSpec],
    activation_dtype: torch.dtype,
    device: torch.device | str,
) -> dict[str, torch.Tensor]:
  """Checks the folder against `specs` and returns name -> tensor on `device`."""
  specs = list(specs)
  entries = st.index_files(st.model_files(model_dir))
  check(specs, entries)
  reader = st.TensorReader(entries)
  out: dict[str, torch.Tensor] = {}
  try:
    for s in specs:
      if s.name not in entries:
        continue
      t = reader.read(s.name)
      out[s.name] = t.to(device=device, dtype=target_dtype(entries[s.name], activation_dtype))
  finally:
    reader.close()
  return out
