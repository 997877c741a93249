"""Typed configuration of the Gemma 2 dense decoder, read from config.json.

Every size and constant comes from the model folder's config.json; this file
only says which key means what and how the keys turn into parts.  The fields
correspond to the reference's experiment-config fields as follows
(simply/config_lib.py:246-342 for the fields, :851-948 for gemma2_2b/9b/27b):

  hidden_size              model_dim
  num_hidden_layers        n_layers
  num_attention_heads      n_heads
  num_key_value_heads      n_kv_heads
  head_dim                 per_head_dim
  intermediate_size        expand_factor * model_dim (simply/model_lib.py:664-667)
  vocab_size               vocab_size
  rms_norm_eps             rms_norm_epsilon (config_lib.py:300)
  rope_theta               RoPE.max_timescale (simply/utils/position_encoding.py:64-66)
  sliding_window           window_size + 1 (config_lib.py:874: window_size excludes the query)
  attn_logit_softcapping   attn_soft_cap (config_lib.py:297)
  final_logit_softcapping  output_logits_soft_cap (config_lib.py:299)
  query_pre_attn_scalar    query_scale ** 2 (simply/model_lib.py:2014-2019, config_lib.py:944)
  hidden_activation        ffn_activation (config_lib.py:292)
  tie_word_embeddings      use_tied_embedding (config_lib.py:287)
  max_position_embeddings  longest context the engine will serve
  layer_types (optional)   block_attn_pattern; absent means local, global, local, ...
                           (config_lib.py:877-880, model_lib.py:2839-2844)
"""

from __future__ import annotations

import dataclasses
import json
import math
import os
from typing import Any

from simply_b200.config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from simply_b200.registry import ARCHITECTURES

_LOCAL = "sliding_attention"
_GLOBAL = "full_attention"

# config.json spelling -> activation registry key.
_ACTIVATION_NAMES = {
    "gelu_pytorch_tanh": "gelu_tanh",
    "gelu_tanh": "gelu_tanh",
    "gelu": "gelu_tanh",  # the reference's 'gelu' is the tanh form (simply/model_lib.py:93-96)
}

_REQUIRED = (
    "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
    "head_dim", "intermediate_size", "vocab_size", "rms_norm_eps", "rope_theta",
    "sliding_window", "attn_logit_softcapping", "final_logit_softcapping",
    "query_pre_attn_scalar", "hidden_activation", "max_position_embeddings",
)


class ConfigError(ValueError):
  """config.json is missing a key or holds a value the engine cannot run."""


@dataclasses.dataclass(frozen=True)
class Gemma2Config:
  hidden_size: int
  num_hidden_layers: int
  num_attention_heads: int
  num_key_value_heads: int
  head_dim: int
  intermediate_size: int
  vocab_size: int
  rms_norm_eps: float
  rope_theta: float
  sliding_window: int
  attn_logit_softcapping: float
  final_logit_softcapping: float
  query_pre_attn_scalar: float
  hidden_activation: str
  max_position_embeddings: int
  tie_word_embeddings: bool = True
  layer_types: tuple[str, ...] = ()
  bos_token_id: int | None = None
  eos_token_id: int | tuple[int, ...] | None = None

  architecture = "Gemma2ForCausalLM"

  # ---- reading and writing ------------------------------------------------
  @classmethod
  def from_dict(cls, d: dict[str, Any]) -> "Gemma2Config":
    missing = [k for k in _REQUIRED if k not in d or d[k] is None]
    if missing:
      raise ConfigError(f"config.json lacks required key(s): {', '.join(missing)}")
    layer_types = tuple(d.get("layer_types") or ())
    eos = d.get("eos_token_id")
    if isinstance(eos, list):
      eos = tuple(int(e) for e in eos)
    cfg = cls(
        hidden_size=int(d["hidden_size"]),
        num_hidden_layers=int(d["num_hidden_layers"]),
        num_attention_heads=int(d["num_attention_heads"]),
        num_key_value_heads=int(d["num_key_value_heads"]),
        head_dim=int(d["head_dim"]),
        intermediate_size=int(d["intermediate_size"]),
        vocab_size=int(d["vocab_size"]),
        rms_norm_eps=float(d["rms_norm_eps"]),
        rope_theta=float(d["rope_theta"]),
        sliding_window=int(d["sliding_window"]),
        attn_logit_softcapping=float(d["attn_logit_softcapping"] or 0.0),
        final_logit_softcapping=float(d["final_logit_softcapping"] or 0.0),
        query_pre_attn_scalar=float(d["query_pre_attn_scalar"]),
        hidden_activation=str(d["hidden_activation"]),
        max_position_embeddings=int(d["max_position_embeddings"]),
        tie_word_embeddings=bool(d.get("tie_word_embeddings", True)),
        layer_types=layer_types,
        bos_token_id=d.get("bos_token_id"),
        eos_token_id=eos,
    )
    cfg.validate()
    return cfg

  def to_dict(self) -> dict[str, Any]:
    d = dataclasses.asdict(self)
    d["architectures"] = [self.architecture]
    d["model_type"] = "gemma2"
    d["layer_types"] = list(self.resolved_layer_types())
    if isinstance(d["eos_token_id"], tuple):
      d["eos_token_id"] = list(d["eos_token_id"])
    # Whole numbers are written as integers, as published config.json files have them (other
    # readers of such a folder insist on an integer query_pre_attn_scalar).
    for key in ("query_pre_attn_scalar", "rope_theta"):
      if float(d[key]).is_integer():
        d[key] = int(d[key])
    return d

  def replace(self, **changes: Any) -> "Gemma2Config":
    cfg = dataclasses.replace(self, **changes)
    cfg.validate()
    return cfg

  # ---- checks ---------------------------------------------------------------
  def validate(self) -> None:
    def need(cond: bool, msg: str) -> None:
      if not cond:
        raise ConfigError(msg)

    for key in ("hidden_size", "num_hidden_layers", "num_attention_heads",
                "num_key_value_heads", "head_dim", "intermediate_size", "vocab_size",
                "sliding_window", "max_position_embeddings"):
      need(getattr(self, key) > 0, f"{key} must be positive, got {getattr(self, key)}")
    need(self.num_attention_heads % self.num_key_value_heads == 0,
         f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
         f"num_key_value_heads ({self.num_key_value_heads})")  # simply/model_lib.py:2032-2036
    need(self.head_dim % 2 == 0, f"head_dim must be even for rotary encoding, got {self.head_dim}")
    need(self.rms_norm_eps > 0, "rms_norm_eps must be positive")
    need(self.rope_theta > 0, "rope_theta must be positive")
    need(self.query_pre_attn_scalar > 0, "query_pre_attn_scalar must be positive")
    need(self.attn_logit_softcapping >= 0 and self.final_logit_softcapping >= 0,
         "soft-capping values must be >= 0 (0 disables)")
    need(self.hidden_activation in _ACTIVATION_NAMES,
         f"unsupported hidden_activation {self.hidden_activation!r}; "
         f"known: {sorted(_ACTIVATION_NAMES)}")
    need(self.tie_word_embeddings,
         "Gemma 2 ties the output layer to the embedding table; "
         "tie_word_embeddings=false is not supported")
    if self.layer_types:
      need(len(self.layer_types) == self.num_hidden_layers,
           f"layer_types has {len(self.layer_types)} entries for "
           f"{self.num_hidden_layers} layers")
      bad = sorted(set(self.layer_types) - {_LOCAL, _GLOBAL})
      need(not bad, f"unknown layer_types entries: {bad}")

  # ---- derived ---------------------------------------------------------------
  def resolved_layer_types(self) -> tuple[str, ...]:
    if self.layer_types:
      return self.layer_types
    return tuple(_LOCAL if i % 2 == 0 else _GLOBAL for i in range(self.num_hidden_layers))

  def model_spec(self) -> ModelSpec:
    norm = {"eps": self.rms_norm_eps, "plus_one": True}
    position = PartSpec("rotary", params={"theta": self.rope_theta, "scale_factor": 1.0})
    layers = []
    for i, kind in enumerate(self.resolved_layer_types()):
      p = f"model.layers.{i}"
      mixer = PartSpec(
          "paged_attention", f"{p}.self_attn",
          {
              "width": self.hidden_size,
              "num_heads": self.num_attention_heads,
              "num_kv_heads": self.num_key_value_heads,
              "head_dim": self.head_dim,
              "query_scale": 1.0 / math.sqrt(self.query_pre_attn_scalar),
              "logit_softcap": self.attn_logit_softcapping,
              "window": self.sliding_window if kind == _LOCAL else None,
              "position": position,
          })
      ffn = PartSpec(
          "gated", f"{p}.mlp",
          {
              "width": self.hidden_size,
              "hidden": self.intermediate_size,
              "activation": _ACTIVATION_NAMES[self.hidden_activation],
          })
      block = PartSpec(
          "sandwich_norm", p,
          {
              "width": self.hidden_size,
              "norm": PartSpec("rms_norm", params=norm),
              "names": {
                  "pre_mixer": "input_layernorm",
                  "post_mixer": "post_attention_layernorm",
                  "pre_feed_forward": "pre_feedforward_layernorm",
                  "post_feed_forward": "post_feedforward_layernorm",
              },
          })
      layers.append(LayerSpec(p, block, mixer, ffn))
    spec = ModelSpec(
        architecture=self.architecture,
        vocab_size=self.vocab_size,
        width=self.hidden_size,
        max_context=self.max_position_embeddings,
        embedding=PartSpec(
            "token_embedding", "model.embed_tokens",
            {"vocab_size": self.vocab_size, "width": self.hidden_size,
             "scale": math.sqrt(self.hidden_size)}),  # simply/utils/module.py:473-481
        layers=tuple(layers),
        run_order=tuple(LayerCall(l.name) for l in layers),
        final_norm=PartSpec("rms_norm", "model.norm", {"width": self.hidden_size, **norm}),
        head=PartSpec("tied_head", "model.embed_tokens",
                      {"logit_softcap": self.final_logit_softcapping}),
    )
    spec.validate()
    return spec


ARCHITECTURES.register(Gemma2Config.architecture, Gemma2Config)
