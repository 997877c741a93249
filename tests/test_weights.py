"""Weights: safetensors by name, one error that lists everything wrong, dtype rule, random mode."""

import json
import os

import numpy as np
import pytest
import torch

from simply_b200.config import load_config, preset
from simply_b200.parts.model import DecoderModel, tensor_specs
from simply_b200.weights import WeightError, load_tensors, random_tensors, write_model_folder
from simply_b200.weights import safetensors_io as st
from tests.reference_ops import ReferenceOps
from tests.tiny_models import write_tiny


def test_writer_is_read_by_the_safetensors_package_and_back(tmp_path):
  from safetensors.torch import load_file, save_file

  tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
             "c": torch.arange(6, dtype=torch.int64).reshape(2, 3), "d": torch.tensor(2.5)}
  st.write_file(str(tmp_path / "mine.safetensors"), tensors, {"k": "v"})
  theirs = load_file(str(tmp_path / "mine.safetensors"))
  save_file(tensors, str(tmp_path / "theirs.safetensors"))
  reader = st.TensorReader(st.index_files([str(tmp_path / "theirs.safetensors")]))
  for name, t in tensors.items():
    assert torch.equal(theirs[name], t)
    got = reader.read(name)
    assert got.dtype == t.dtype and torch.equal(got, t)


def test_random_mode_writes_a_loadable_folder(tmp_path):
  folder = write_tiny("b", tmp_path, "bfloat16")
  assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
  cfg = load_config(folder)
  assert cfg.hidden_size == 96
  specs = tensor_specs(cfg.model_spec())
  t = load_tensors(folder, specs, torch.bfloat16, "cpu")
  assert t["model.embed_tokens.weight"].shape == (1000, 96)
  assert t["model.layers.4.self_attn.q_proj.weight"].shape == (6 * 32, 96)
  assert t["model.layers.0.mlp.down_proj.weight"].shape == (96, 320)
  assert all(v.dtype == torch.bfloat16 for v in t.values())
  assert abs(t["model.layers.1.mlp.up_proj.weight"].float().std().item() - 0.05) < 0.005
  assert abs(t["model.layers.2.input_layernorm.weight"].float().std().item() - 0.2) < 0.06
  # same seed, same weights; another seed, other weights
  again = load_tensors(write_tiny("b", tmp_path / "x", "bfloat16"), specs, torch.bfloat16, "cpu")
  assert all(torch.equal(again[k], t[k]) for k in t)
  other = random_tensors(specs, 5, dtype=torch.bfloat16)
  assert not torch.equal(other["model.embed_tokens.weight"], t["model.embed_tokens.weight"])


def test_dtype_rule(tmp_path):
  folder = write_tiny("a", tmp_path, "bfloat16")
  specs = tensor_specs(load_config(folder).model_spec())
  # a folder whose norm scales are stored in 32 bits
  entries = st.index_files(st.model_files(folder))
  reader = st.TensorReader(entries)
  tensors = {n: reader.read(n) for n in entries}
  reader.close()
  name = "model.layers.0.input_layernorm.weight"
  tensors[name] = tensors[name].float()
  st.write_file(os.path.join(folder, "model.safetensors"), tensors)
  bf = load_tensors(folder, specs, torch.bfloat16, "cpu")
  assert bf[name].dtype == torch.float32  # stored in 32 bits, stays so
  assert bf["model.norm.weight"].dtype == torch.bfloat16
  f32 = load_tensors(folder, specs, torch.float32, "cpu")
  assert all(v.dtype == torch.float32 for v in f32.values())
  assert torch.equal(f32["model.norm.weight"], bf["model.norm.weight"].float())


def test_a_folder_stored_in_float32_is_narrowed_to_the_activation_dtype(tmp_path, capsys):
  """simply/utils/checkpoint_lib.py:658-670: wider floats are restored in the activation dtype.
  Matrices become bfloat16 (and equal the bfloat16 folder's), norm scales stay as stored."""
  narrow = write_tiny("a", tmp_path / "n", "bfloat16")
  wide = write_tiny("a", tmp_path / "w", "float32")
  specs = tensor_specs(load_config(wide).model_spec())
  a = load_tensors(narrow, specs, torch.bfloat16, "cpu")
  b = load_tensors(wide, specs, torch.bfloat16, "cpu")
  assert "narrowed to bfloat16" in capsys.readouterr().err
  for name, t in b.items():
    if name.endswith("norm.weight") or "layernorm" in name:
      assert t.dtype == torch.float32
      assert torch.equal(t.to(torch.bfloat16), a[name])
    else:
      assert t.dtype == torch.bfloat16 and torch.equal(t, a[name]), name
  kept = load_tensors(wide, specs, torch.bfloat16, "cpu", keep_float32=True)
  assert all(t.dtype == torch.float32 for t in kept.values())
  # a part may declare a matrix of its own as precision-critical
  import dataclasses
  name = "model.layers.0.mlp.down_proj.weight"
  special = [dataclasses.replace(s, precision="stored") if s.name == name else s for s in specs]
  assert load_tensors(wide, special, torch.bfloat16, "cpu")[name].dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
  folder = write_tiny("a", tmp_path, "bfloat16")
  specs = tensor_specs(load_config(folder).model_spec())
  entries = st.index_files(st.model_files(folder))
  reader = st.TensorReader(entries)
  tensors = {n: reader.read(n) for n in entries}
  reader.close()
  del tensors["model.norm.weight"]
  del tensors["model.layers.1.mlp.up_proj.weight"]
  tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
  tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(32, 64, dtype=torch.bfloat16)
  tensors["model.layers.1.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
  st.write_file(os.path.join(folder, "model.safetensors"), tensors)
  with pytest.raises(WeightError) as e:
    load_tensors(folder, specs, torch.bfloat16, "cpu")
  err = e.value
  assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
  assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
  assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (16, 64), (32, 64))]
  assert err.wrong_kind[0][0] == "model.layers.1.input_layernorm.weight"
  msg = str(err)
  for needle in ("missing tensors (2)", "unexpected tensors (1)", "[32, 64]", "[16, 64]", "rotary_emb"):
    assert needle in msg


def test_tied_table_may_be_repeated_as_lm_head(tmp_path):
  folder = write_tiny("a", tmp_path, "bfloat16")
  specs = tensor_specs(load_config(folder).model_spec())
  entries = st.index_files(st.model_files(folder))
  reader = st.TensorReader(entries)
  tensors = {n: reader.read(n) for n in entries}
  reader.close()
  tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
  st.write_file(os.path.join(folder, "model.safetensors"), tensors)
  loaded = load_tensors(folder, specs, torch.bfloat16, "cpu")
  DecoderModel(load_config(folder).model_spec()).bind(loaded, ReferenceOps(torch.bfloat16))  # a copy: accepted
  # ... but not another table under that name
  tensors["lm_head.weight"][3, 5] += 1.0
  st.write_file(os.path.join(folder, "model.safetensors"), tensors)
  loaded = load_tensors(folder, specs, torch.bfloat16, "cpu")
  with pytest.raises(WeightError, match="lm_head.weight differs"):
    DecoderModel(load_config(folder).model_spec()).bind(loaded, ReferenceOps(torch.bfloat16))


def test_broken_files(tmp_path):
  (tmp_path / "model.safetensors").write_bytes(b"\x05\x00")
  with pytest.raises(st.SafetensorsError, match="too short"):
    st.index_files(st.model_files(str(tmp_path)))
  (tmp_path / "model.safetensors").write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
  with pytest.raises(st.SafetensorsError, match="header length"):
    st.index_files(st.model_files(str(tmp_path)))
  with pytest.raises(st.SafetensorsError, match="no \\*.safetensors"):
    st.model_files(str(tmp_path / "nowhere"))
  a = {"x": torch.zeros(2)}
  st.write_file(str(tmp_path / "m1.safetensors"), a)
  st.write_file(str(tmp_path / "m2.safetensors"), a)
  with pytest.raises(st.SafetensorsError, match="appears in both"):
    st.index_files([str(tmp_path / "m1.safetensors"), str(tmp_path / "m2.safetensors")])


def test_two_parts_may_not_claim_one_tensor():
  from simply_b200.config.model_spec import LayerSpec
  import dataclasses
  spec = preset("gemma2-tiny-a").model_spec()
  l0 = spec.layers[0]
  clash = dataclasses.replace(spec.layers[1], mixer=dataclasses.replace(spec.layers[1].mixer, prefix=l0.mixer.prefix))
  bad = dataclasses.replace(spec, layers=(l0, clash))
  with pytest.raises(ValueError, match="same tensor"):
    DecoderModel(bad).tensor_specs()
