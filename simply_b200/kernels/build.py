"""Builds the CUDA sources under simply_b200/csrc into one shared library and loads it.

The library is plain `extern "C"` functions taking raw pointers and a stream,
called through ctypes, so a build is a few nvcc invocations (seconds each) and
needs no Python headers.  It is compiled for sm_100a only.  The result lives in
`simply_b200/csrc/_build/` (or, when that is not writable, under the system's
temporary directory) next to a stamp of the sources' hash; a changed source or
flag triggers a rebuild at the next load.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libsimply_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


class KernelBuildError(RuntimeError):
  pass


# Sources that are compiled once per head size (-DSB_HEAD_DIM=N) into libraries of their own.
PER_HEAD_DIM = ("attention_mma.cu", "attention_tc.cu", "attention_tc_pair.cu")


def sources() -> list[str]:
  return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC)
                if f.endswith(".cu") and f not in PER_HEAD_DIM)


def _headers() -> list[str]:
  return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _digest(srcs: list[str] | None = None, extra: str = "") -> str:
  h = hashlib.sha256()
  h.update(extra.encode())
  for path in (sources() if srcs is None else srcs) + _headers():
    h.update(os.path.basename(path).encode())
    with open(path, "rb") as f:
      h.update(f.read())
  h.update(" ".join(NVCC_FLAGS).encode())
  return h.hexdigest()[:16]


def _find_nvcc() -> str:
  for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
    if cand and os.path.isfile(cand):
      return cand
  raise KernelBuildError("nvcc not found (set NVCC or put it on PATH); the engine has no other backend")


def _build_dir() -> str:
  d = os.path.join(CSRC, "_build")
  try:
    os.makedirs(d, exist_ok=True)
    probe = os.path.join(d, f".w{os.getpid()}")
    with open(probe, "w"):
      pass
    os.remove(probe)
    return d
  except OSError:
    d = os.path.join(tempfile.gettempdir(), f"simply_b200_build_{os.getuid()}")
    os.makedirs(d, exist_ok=True)
    return d


def _say(msg: str) -> None:
  print(f"[simply_b200] {msg}", file=sys.stderr, flush=True)


def build(verbose: bool = True, force: bool = False) -> str:
  """Compiles the core library if it is missing or stale; returns its path."""
  return _build(sources(), LIB_NAME, [], verbose, force)


def attention_lib_name(head_dim: int) -> str:
  return f"libsimply_b200_attn_hd{head_dim}.so"


def build_attention(head_dim: int, verbose: bool = True, force: bool = False) -> str:
  """Compiles the tensor-core attention kernels for one head size; returns the library's path."""
  if head_dim % 16 or not 16 <= head_dim <= 256:
    raise KernelBuildError(f"tensor-core attention takes head sizes 16, 32, ..., 256; got {head_dim}")
  srcs = [os.path.join(CSRC, f) for f in PER_HEAD_DIM]
  return _build(srcs, attention_lib_name(head_dim), [f"-DSB_HEAD_DIM={head_dim}"], verbose, force)


def _build(srcs: list[str], lib_name: str, defines: list[str], verbose: bool, force: bool) -> str:
  out_dir = _build_dir()
  lib = os.path.join(out_dir, lib_name)
  stamp = os.path.join(out_dir, lib_name + ".stamp")
  digest = _digest(srcs, " ".join(defines))
  if not force and os.path.isfile(lib) and os.path.isfile(stamp):
    with open(stamp) as f:
      if f.read().strip() == digest:
        return lib
  nvcc = _find_nvcc()
  if verbose:
    _say(f"compiling {lib_name} ({len(srcs)} CUDA source(s), sm_100a) into {out_dir} (first use only)")
  t0 = time.time()
  procs = []
  for src in srcs:
    obj = os.path.join(out_dir, lib_name[:-3] + "." + os.path.basename(src)[:-3] + ".o")
    cmd = [nvcc, *NVCC_FLAGS, *defines, "-I", CSRC, "-c", src, "-o", obj]
    procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
  objs = []
  pending = list(procs)
  last = time.time()
  while pending:
    for item in list(pending):
      src, obj, p = item
      if p.poll() is not None:
        pending.remove(item)
        out = p.stdout.read().decode(errors="replace")
        if p.returncode != 0:
          for _, _, q in pending:
            q.kill()
          raise KernelBuildError(f"nvcc failed on {src}:\n{out}")
        objs.append(obj)
        if verbose:
          _say(f"  compiled {os.path.basename(src)} ({time.time() - t0:.0f} s)")
    if pending:
      time.sleep(0.2)
      if verbose and time.time() - last > 10:
        _say(f"  still compiling {len(pending)} file(s) ... {time.time() - t0:.0f} s")
        last = time.time()
  tmp = lib + f".{os.getpid()}.tmp"
  link = [nvcc, "-shared", "-o", tmp, *sorted(objs), "-gencode", "arch=compute_100a,code=sm_100a",
          "-lcudart", "-ldl"]
  r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
  if r.returncode != 0:
    raise KernelBuildError(f"linking {lib_name} failed:\n{r.stdout.decode(errors='replace')}")
  os.replace(tmp, lib)
  with open(stamp, "w") as f:
    f.write(digest)
  if verbose:
    _say(f"built {lib} in {time.time() - t0:.0f} s")
  return lib


def load() -> ctypes.CDLL:
  """Builds if needed and loads the core library; raises if that is not possible."""
  global _lib
  with _lock:
    if _lib is None:
      _lib = ctypes.CDLL(build())
    return _lib


_attention_libs: dict[int, ctypes.CDLL] = {}


def load_attention(head_dim: int) -> ctypes.CDLL:
  """Builds if needed and loads the attention library of one head size."""
  with _lock:
    lib = _attention_libs.get(head_dim)
    if lib is None:
      lib = ctypes.CDLL(build_attention(head_dim))
      _attention_libs[head_dim] = lib
    return lib
