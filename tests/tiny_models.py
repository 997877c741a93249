"""The tests' tiny configurations and helpers that write them as model folders.

Tiny A and tiny B differ in every size and option: layers, width, head counts
and grouping, head size, feed-forward width, vocabulary, rotary base, window,
both soft caps, the query scale and the norms' eps.
"""

import os

from simply_b200.config import preset
from simply_b200.weights import write_model_folder

# name -> (preset, seed, matrix_std, scale_std)
TINY = {
    "a": ("gemma2-tiny-a", 0, 0.02, 0.1),
    "b": ("gemma2-tiny-b", 2, 0.05, 0.2),
}


def write_tiny(which: str, root, dtype: str = "bfloat16", **changes) -> str:
  name, seed, matrix_std, scale_std = TINY[which]
  cfg = preset(name)
  if changes:
    cfg = cfg.replace(**changes)
  out = os.path.join(str(root), f"tiny_{which}_{dtype}")
  write_model_folder(cfg, seed, out, matrix_std=matrix_std, scale_std=scale_std, dtype=dtype)
  return out
