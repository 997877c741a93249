"""The command line `python -m simply_b200`, run as a user runs it (a child process).

Its flags carry the names of the reference's serving flags (simply/serving/common_flags.py:19-132)
and of its evaluation entry point (simply/eval/page_decode_eval.py:50-109, :122)."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest

from simply_b200.config import load_config
from tests.plain.gemma2_plain import PlainGemma2
from tests.tiny_models import TINY, write_tiny

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def cli(*args, ok=True):
  env = dict(os.environ, PYTHONPATH=REPO + os.pathsep + os.environ.get("PYTHONPATH", ""))
  p = subprocess.run([sys.executable, "-m", "simply_b200", *args], capture_output=True, text=True, env=env,
                     cwd=REPO, timeout=900)
  if ok:
    assert p.returncode == 0, p.stderr[-2000:]
  return p


def json_lines(text):
  return [json.loads(line) for line in text.splitlines() if line.startswith("{")]


def test_write_model_dir_writes_a_folder_other_readers_accept(tmp_path):
  out = str(tmp_path / "m")
  p = cli("--experiment_config", "gemma2-tiny-b", "--write_model_dir", out, "--model_seed", "2",
          "--matrix_std", "0.05", "--scale_std", "0.2")
  assert json_lines(p.stdout) == [{"wrote": out}]
  assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
  with open(os.path.join(out, "config.json")) as f:
    d = json.load(f)
  # whole numbers are integers in the file, as in published folders
  assert d["query_pre_attn_scalar"] == 48 and isinstance(d["query_pre_attn_scalar"], int)
  assert isinstance(d["rope_theta"], int) and isinstance(d["rms_norm_eps"], float)
  assert d["architectures"] == ["Gemma2ForCausalLM"] and len(d["layer_types"]) == 5
  assert load_config(out) == load_config(write_tiny("b", tmp_path / "direct"))
  # the same weights as the library call with these arguments
  a = PlainGemma2(out).tensors
  b = PlainGemma2(write_tiny("b", tmp_path / "again")).tensors
  assert sorted(a) == sorted(b) and all(np.array_equal(a[k], b[k]) for k in a)


def test_config_overlay_as_json_and_as_a_file(tmp_path):
  overlay = {"num_hidden_layers": 3, "sliding_window": 5, "query_pre_attn_scalar": 20.5}
  out1, out2 = str(tmp_path / "a"), str(tmp_path / "b")
  cli("--experiment_config", "gemma2-tiny-a", "--write_model_dir", out1, "--config_overlay", json.dumps(overlay))
  path = tmp_path / "overlay.json"
  path.write_text(json.dumps(overlay))
  cli("--experiment_config", "gemma2-tiny-a", "--write_model_dir", out2, "--config_overlay", str(path))
  c1, c2 = load_config(out1), load_config(out2)
  assert c1 == c2 and c1.num_hidden_layers == 3 and c1.sliding_window == 5 and c1.query_pre_attn_scalar == 20.5
  assert c1.hidden_size == 64  # what the overlay does not name stays
  with open(os.path.join(out1, "config.json")) as f:
    assert json.load(f)["query_pre_attn_scalar"] == 20.5


def test_usage_errors():
  assert cli("--write_model_dir", "/nonexistent/x", ok=False).returncode != 0  # no --experiment_config
  p = cli("--experiment_config", "no-such-config", "--write_model_dir", "/nonexistent/x", ok=False)
  assert p.returncode != 0 and "unknown preset" in p.stderr
  p = cli("--ckpt_dir", "/nonexistent/x", ok=False)
  assert p.returncode != 0 and "prompt_ids" in p.stderr


@pytest.mark.gpu
def test_greedy_and_sampled_generation_from_a_folder(tmp_path):
  folder = write_tiny("b", tmp_path)
  plain = PlainGemma2(folder)
  rng = np.random.default_rng(4)
  prompts = [rng.integers(0, plain.cfg["vocab_size"], n).tolist() for n in (3, 19, 41)]
  ids = ";".join(",".join(str(t) for t in p) for p in prompts)
  common = ("--ckpt_dir", folder, "--activation_dtype", "float32", "--page_size", "8", "--batch_size", "2",
            "--max_seq_len", "128", "--max_decode_steps", "9")
  p = cli(*common, "--prompt_ids", ids, "--temperature", "0")
  got = json_lines(p.stdout)
  assert [g["input_token_ids"] for g in got] == prompts
  assert [g["output_token_ids"] for g in got] == [plain.greedy(q, 9) for q in prompts]
  assert all(g["finish_reason"] == "max_decode_steps" and g["is_truncated"] for g in got)
  # sampled, prompts from a file, steps in bursts, a small token budget; request i samples with seed + i
  path = tmp_path / "prompts.txt"
  path.write_text("\n".join(" ".join(str(t) for t in q) for q in prompts) + "\n")
  p = cli(*common, "--prompt_file", str(path), "--temperature", "0.8", "--top_k", "40", "--top_p", "0.95",
          "--seed", "7", "--intermediate_steps", "4", "--max_num_issue_tokens", "16")
  got = json_lines(p.stdout)
  want = [plain.sample(q, 9, 0.8, 7 + i, top_k=40, top_p=0.95) for i, q in enumerate(prompts)]
  assert [g["output_token_ids"] for g in got] == want


@pytest.mark.gpu
def test_random_weights_of_a_named_configuration():
  p = cli("--experiment_config", "gemma2-tiny-a", "--random_weights", "--prompt_ids", "5,6,7", "--temperature", "0",
          "--max_decode_steps", "4", "--max_seq_len", "64", "--config_overlay", '{"num_hidden_layers": 1}')
  got = json_lines(p.stdout)
  assert len(got) == 1 and len(got[0]["output_token_ids"]) == 4
