"""Minimal reader and writer of the safetensors container.

Layout of a file: 8 bytes little-endian header length N, N bytes of JSON
`{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}`,
then one byte buffer that the offsets index.  Tensors are read by name through
a memory map, so a tensor that is not asked for costs nothing.

The reference reads safetensors only in its offline converter
(simply/tools/hf_to_orbax.py:50-85: open every `model*.safetensors`, reject
duplicate keys); serving restores Orbax trees (simply/utils/checkpoint_lib.py:690-809).
This engine serves straight from the safetensors folder.
"""

from __future__ import annotations

import dataclasses
import glob
import json
import mmap
import os
import struct
from typing import Iterable

import numpy as np
import torch

# safetensors dtype code -> (numpy dtype used to view the bytes, torch dtype).
_DTYPES = {
    "F64": (np.float64, torch.float64),
    "F32": (np.float32, torch.float32),
    "F16": (np.float16, torch.float16),
    "BF16": (np.uint16, torch.bfloat16),
    "I64": (np.int64, torch.int64),
    "I32": (np.int32, torch.int32),
    "I16": (np.int16, torch.int16),
    "I8": (np.int8, torch.int8),
    "U8": (np.uint8, torch.uint8),
    "BOOL": (np.bool_, torch.bool),
}
_CODE_OF_TORCH = {v[1]: k for k, v in _DTYPES.items()}


@dataclasses.dataclass(frozen=True)
class TensorEntry:
  name: str
  dtype: str  # safetensors code, e.g. "BF16"
  shape: tuple[int, ...]
  file: str
  begin: int  # byte offsets inside the file
  end: int

  @property
  def is_float(self) -> bool:
    return self.dtype in ("F64", "F32", "F16", "BF16")

  @property
  def is_32bit_float(self) -> bool:
    return self.dtype in ("F32", "F64")


class SafetensorsError(ValueError):
  pass


def _read_header(path: str) -> tuple[dict, int]:
  with open(path, "rb") as f:
    head = f.read(8)
    if len(head) != 8:
      raise SafetensorsError(f"{path}: too short to be a safetensors file")
    (n,) = struct.unpack("<Q", head)
    size = os.path.getsize(path)
    if n <= 0 or 8 + n > size:
      raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
    try:
      header = json.loads(f.read(n))
    except json.JSONDecodeError as e:
      raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
  return header, 8 + n


def index_files(paths: Iterable[str]) -> dict[str, TensorEntry]:
  """Reads the headers of `paths` and returns name -> entry; duplicate names are an error."""
  entries: dict[str, TensorEntry] = {}
  for path in paths:
    header, base = _read_header(path)
    size = os.path.getsize(path)
    for name, meta in header.items():
      if name == "__metadata__":
        continue
      if name in entries:
        raise SafetensorsError(f"tensor {name!r} appears in both {entries[name].file} and {path}")
      dtype = meta["dtype"]
      if dtype not in _DTYPES:
        raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype}")
      b, e = meta["data_offsets"]
      shape = tuple(int(s) for s in meta["shape"])
      want = int(np.prod(shape, dtype=np.int64)) * np.dtype(_DTYPES[dtype][0]).itemsize
      if e - b != want or base + e > size:
        raise SafetensorsError(
            f"{path}: tensor {name!r} claims bytes [{b}, {e}) for shape {shape} {dtype}; "
            f"expected {want} bytes within a {size}-byte file")
      entries[name] = TensorEntry(name, dtype, shape, path, base + b, base + e)
  return entries


def model_files(model_dir: str) -> list[str]:
  files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
  if not files:
    raise SafetensorsError(f"no *.safetensors file in {model_dir!r}")
  return files


class TensorReader:
  """Reads tensors by name from a set of memory-mapped safetensors files."""

  def __init__(self, entries: dict[str, TensorEntry]):
    self.entries = entries
    self._maps: dict[str, mmap.mmap] = {}

  def _map(self, path: str) -> mmap.mmap:
    m = self._maps.get(path)
    if m is None:
      with open(path, "rb") as f:
        m = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
      self._maps[path] = m
    return m

  def read(self, name: str) -> torch.Tensor:
    """Returns the tensor as stored (a CPU copy, in its stored dtype)."""
    e = self.entries[name]
    np_dtype, torch_dtype = _DTYPES[e.dtype]
    count = int(np.prod(e.shape, dtype=np.int64))
    arr = np.frombuffer(self._map(e.file), dtype=np_dtype, count=count, offset=e.begin)
    t = torch.from_numpy(arr.copy())
    if e.dtype == "BF16":
      t = t.view(torch.bfloat16)
    return t.reshape(e.shape)

  def close(self) -> None:
    for m in self._maps.values():
      m.close()
    self._maps.clear()


def write_file(path: str, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
  """Writes `tensors` (CPU or device; any listed dtype) as one safetensors file."""
  header: dict = {}
  if metadata:
    header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
  offset = 0
  blobs = []
  for name in sorted(tensors):
    t = tensors[name].detach().cpu().contiguous()
    if t.dtype not in _CODE_OF_TORCH:
      raise SafetensorsError(f"cannot write tensor {name!r} of dtype {t.dtype}")
    raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
    header[name] = {
        "dtype": _CODE_OF_TORCH[t.dtype],
        "shape": list(t.shape),
        "data_offsets": [offset, offset + len(raw)],
    }
    offset += len(raw)
    blobs.append(raw)
  head = json.dumps(header, separators=(",", ":")).encode()
  head += b" " * (-len(head) % 8)
  tmp = path + ".tmp"
  with open(tmp, "wb") as f:
    f.write(struct.pack("<Q", len(head)))
    f.write(head)
    for raw in blobs:
      f.write(raw)
  os.replace(tmp, path)
