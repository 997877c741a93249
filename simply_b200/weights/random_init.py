"""Random-weights mode: fills a model's tensors from a seed and writes a model folder.

The reference initialises with `model.init(jax.random.key(seed))`: Xavier-uniform
linears, Lecun-normal embedding, zero `(1+w)` norm scales
(simply/utils/initializer.py:90-153, simply/model_lib.py:130-152, :2854-2872).
This engine's benchmark and test configurations prescribe their own law instead:
matrices and embeddings N(0, matrix_std), norm scales N(0, scale_std).  Each tensor
draws from its own generator keyed by (seed, position of the tensor's name in the
sorted name list), so the values do not depend on the order of generation.
"""

from __future__ import annotations

import json
import os
from typing import Iterable

import torch

from simply_b200.weights import safetensors_io as st
from simply_b200.weights.loader import TensorSpec

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def random_tensors(
    specs: Iterable[TensorSpec],
    seed: int,
    *,
    matrix_std: float = 0.02,
    scale_std: float = 0.0,
    dtype: torch.dtype = torch.bfloat16,
    device: torch.device | str = "cpu",
) -> dict[str, torch.Tensor]:
  """Draws every non-optional tensor of `specs`; values are generated in float32 then cast."""
  specs = sorted((s for s in specs if not s.optional), key=lambda s: s.name)
  device = torch.device(device)
  out: dict[str, torch.Tensor] = {}
  for i, s in enumerate(specs):
    gen = torch.Generator(device=device)
    gen.manual_seed((int(seed) << 20) + i)
    if s.kind == "table":
      out[s.name] = torch.zeros(s.shape, dtype=torch.int32, device=device)
      continue
    std = scale_std if s.kind == "scale" else matrix_std
    if std == 0.0:
      t = torch.zeros(s.shape, dtype=torch.float32, device=device)
    else:
      t = torch.randn(s.shape, generator=gen, dtype=torch.float32, device=device) * std
    out[s.name] = t.to(dtype)
  return out


def write_model_folder(
    config,
    seed: int,
    out_dir: str,
    *,
    matrix_std: float = 0.02,
    scale_std: float = 0.0,
    dtype: str = "bfloat16",
    device: torch.device | str = "cpu",
) -> str:
  """Writes config.json and model.safetensors for `config` (an architecture config object).
  `device` is where the values are drawn (each device's generator has its own sequence)."""
  from simply_b200.parts.model import tensor_specs  # parts import weights.loader; avoid a cycle

  if dtype not in _TORCH_DTYPES:
    raise ValueError(f"dtype must be one of {sorted(_TORCH_DTYPES)}, got {dtype!r}")
  os.makedirs(out_dir, exist_ok=True)
  tensors = random_tensors(
      tensor_specs(config.model_spec()), seed, matrix_std=matrix_std, scale_std=scale_std,
      dtype=_TORCH_DTYPES[dtype], device=device)
  tensors = {name: t.cpu() for name, t in tensors.items()}
  with open(os.path.join(out_dir, "config.json"), "w") as f:
    json.dump(config.to_dict(), f, indent=1)
  st.write_file(
      os.path.join(out_dir, "model.safetensors"), tensors,
      metadata={"format": "pt", "seed": str(seed), "matrix_std": str(matrix_std),
                "scale_std": str(scale_std)})
  return out_dir
