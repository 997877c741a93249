"""Writes tests/golden/plain_tiny.npz: logits of the plain NumPy model on the two tiny
configurations, so that a later change to tests/plain/ that alters its arithmetic shows.

These are the plain implementation's own outputs.  The reference's model code cannot be
imported here (no JAX), so nothing in this folder comes from running google-deepmind/simply.

  python tests/golden/make_golden.py
"""

import os
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from tests.plain.gemma2_plain import PlainGemma2  # noqa: E402
from tests.tiny_models import write_tiny  # noqa: E402

PROMPTS = {"a": [3, 141, 59, 26, 53, 58, 97, 93, 23, 84, 62, 64], "b": [314, 159, 265, 358, 979, 323, 846, 264, 338, 327]}


def compute():
  out = {}
  with tempfile.TemporaryDirectory() as tmp:
    for which, prompt in PROMPTS.items():
      model = PlainGemma2(write_tiny(which, tmp, "bfloat16"), np.float64)
      out[which] = model.forward(prompt).astype(np.float32)
  return out


if __name__ == "__main__":
  np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "plain_tiny.npz"), **compute())
  print("wrote plain_tiny.npz")
