"""Configuration: config.json keys -> typed config -> model description; registries."""

import json

import pytest

from simply_b200 import config as cfg_lib
from simply_b200.config import ConfigError, EngineConfig, Gemma2Config, preset, preset_dict
from simply_b200.registry import ARCHITECTURES, Registry


def test_presets_match_the_published_shapes():
  c = preset("gemma2-2b")
  assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
          c.intermediate_size, c.vocab_size, c.sliding_window) == (2304, 26, 8, 4, 256, 9216, 256000, 4096)
  assert preset("gemma2-27b").query_pre_attn_scalar == 144  # width / heads, not the head size
  assert set(cfg_lib.preset_names()) >= {"gemma2-2b", "gemma2-9b", "gemma2-27b", "gemma2-tiny-a", "gemma2-tiny-b"}


def test_tiny_configs_differ_in_every_size_and_option():
  a, b = preset_dict("gemma2-tiny-a"), preset_dict("gemma2-tiny-b")
  for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
              "intermediate_size", "vocab_size", "rms_norm_eps", "rope_theta", "sliding_window",
              "attn_logit_softcapping", "final_logit_softcapping", "query_pre_attn_scalar"):
    assert a[key] != b[key], key
  assert a["num_attention_heads"] // a["num_key_value_heads"] != b["num_attention_heads"] // b["num_key_value_heads"]


def test_model_spec_takes_every_constant_from_the_config():
  d = preset_dict("gemma2-tiny-b")
  spec = cfg_lib.config_from_dict(d).model_spec()
  assert spec.vocab_size == 1000 and spec.width == 96 and len(spec.layers) == 5
  windows = [l.mixer.params["window"] for l in spec.layers]
  assert windows == [16, None, 16, None, 16]  # local, global, local, ...
  m = spec.layers[0].mixer.params
  assert m["query_scale"] == pytest.approx(48 ** -0.5) and m["logit_softcap"] == 20.0
  assert m["position"].params["theta"] == 500000.0
  assert spec.layers[0].block.params["norm"].params["eps"] == 1e-5
  assert spec.head.params["logit_softcap"] == 10.0
  assert [c.layer for c in spec.run_order] == [l.name for l in spec.layers]
  # changing a key changes the spec: nothing is hard-wired
  d2 = dict(d, rope_theta=777.0, sliding_window=5, layer_types=["full_attention"] * 4 + ["sliding_attention"])
  spec2 = cfg_lib.config_from_dict(d2).model_spec()
  assert [l.mixer.params["window"] for l in spec2.layers] == [None] * 4 + [5]
  assert spec2.layers[0].mixer.params["position"].params["theta"] == 777.0


def test_round_trip_through_json(tmp_path):
  c = preset("gemma2-tiny-a")
  (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
  assert cfg_lib.load_config(str(tmp_path)) == c.replace(layer_types=c.resolved_layer_types())


@pytest.mark.parametrize("change,needle", [
    ({"head_dim": None}, "head_dim"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_activation": "swish"}, "hidden_activation"),
    ({"tie_word_embeddings": False}, "tie"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"layer_types": ["x", "y"]}, "unknown layer_types"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"architectures": ["NoSuchModel"]}, "unknown name"),
    ({"architectures": []}, "architectures"),
])
def test_bad_configs_are_refused(change, needle):
  d = dict(preset_dict("gemma2-tiny-a"), **change)
  if change.get("head_dim", 0) is None:
    del d["head_dim"]
  with pytest.raises(ConfigError, match=needle):
    cfg_lib.config_from_dict(d)


def test_missing_config_file(tmp_path):
  with pytest.raises(ConfigError, match="config.json"):
    cfg_lib.load_config(str(tmp_path))


def test_registry():
  r = Registry("thing")
  r.register("a", 1)

  @r.register("b")
  def b():
    return 2

  assert r.get("a") == 1 and r.get("b") is b and r.keys() == ["a", "b"] and "a" in r
  with pytest.raises(ValueError, match="duplicate"):
    r.register("a", 3)
  r.register("a", 3, replace=True)
  assert r.get("a") == 3
  with pytest.raises(KeyError, match="registered: a, b"):
    r.get("c")
  r.unregister("a")
  assert "a" not in r
  assert ARCHITECTURES.get("Gemma2ForCausalLM") is Gemma2Config


def test_engine_config():
  e = EngineConfig(activation_dtype="bf16", page_size=16, batch_size=3).resolved(1000)
  assert e.activation_dtype == "bfloat16" and e.max_seq_len == 1000
  assert e.max_cache_tokens == 3 * 1008 and e.max_num_issue_tokens == 2048
  with pytest.raises(ValueError):
    EngineConfig(activation_dtype="float16")
  with pytest.raises(ValueError):
    EngineConfig(page_size=0)
  with pytest.raises(ValueError, match="exceeds"):
    EngineConfig(max_seq_len=2000).resolved(1000)
