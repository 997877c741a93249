"""Configuration: config.json -> typed architecture config -> neutral ModelSpec."""

from __future__ import annotations

import json
import os
from typing import Any

from simply_b200.config.engine_config import EngineConfig
from simply_b200.config.gemma2 import ConfigError, Gemma2Config
from simply_b200.config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from simply_b200.registry import ARCHITECTURES

_PRESET_DIR = os.path.join(os.path.dirname(__file__), "presets")


def read_config_json(model_dir: str) -> dict[str, Any]:
  path = os.path.join(model_dir, "config.json")
  if not os.path.isfile(path):
    raise ConfigError(f"no config.json in {model_dir!r}")
  with open(path) as f:
    return json.load(f)


def config_from_dict(d: dict[str, Any]):
  """Picks the config class by config.json's `architectures[0]` and builds it."""
  archs = d.get("architectures")
  if not archs:
    raise ConfigError("config.json has no 'architectures' entry")
  try:
    cls = ARCHITECTURES.get(archs[0])
  except KeyError as e:
    raise ConfigError(str(e)) from None
  return cls.from_dict(d)


def load_config(model_dir: str):
  return config_from_dict(read_config_json(model_dir))


def preset_names() -> list[str]:
  return sorted(f[:-5] for f in os.listdir(_PRESET_DIR) if f.endswith(".json"))


def preset_dict(name: str) -> dict[str, Any]:
  """config.json contents of a named preset (data files under config/presets)."""
  path = os.path.join(_PRESET_DIR, name + ".json")
  if not os.path.isfile(path):
    raise ConfigError(f"unknown preset {name!r}; known: {', '.join(preset_names())}")
  with open(path) as f:
    return json.load(f)


def preset(name: str):
  return config_from_dict(preset_dict(name))


__all__ = [
    "ConfigError", "EngineConfig", "Gemma2Config", "LayerCall", "LayerSpec", "ModelSpec",
    "PartSpec", "config_from_dict", "load_config", "preset", "preset_dict", "preset_names",
    "read_config_json",
]
