"""Command line: generate tokens from a model folder, or write a random-weights model folder.

  python -m simply_b200 --ckpt_dir DIR --prompt_ids "2,651,9456;2,1841" --temperature 0 --max_decode_steps 32
  python -m simply_b200 --experiment_config gemma2-tiny-a --write_model_dir /tmp/m --model_seed 0

Flag names and meanings follow google-deepmind/simply's serving flags where it has them
(simply/serving/common_flags.py:19-132): --experiment_config, --ckpt_dir, --batch_size,
--activation_dtype, --max_seq_len, --max_decode_steps, --page_size, --temperature, --top_k,
--top_p, --intermediate_steps, --max_num_issue_tokens; --seed is its evaluation script's
(simply/eval/page_decode_eval.py:50-109), --model_seed its config field (simply/config_lib.py:863).
Token ids in, token ids out: one JSON object per prompt on standard output.
"""

from __future__ import annotations

import json
import os
import sys

from absl import app, flags

FLAGS = flags.FLAGS

flags.DEFINE_string("ckpt_dir", None, "Model folder: config.json and *.safetensors.")
flags.DEFINE_string("experiment_config", None,
                    "Name of a registered configuration (a preset); with --write_model_dir or "
                    "--random_weights it names the model to fill with random weights.")
flags.DEFINE_string("config_overlay", None,
                    "JSON object (or a file holding one) of config.json keys that replace the named "
                    "configuration's values (simply/main.py:38-42).")
flags.DEFINE_string("write_model_dir", None, "Write a random-weights model folder here and exit.")
flags.DEFINE_bool("random_weights", False, "Run --experiment_config with random weights drawn on the GPU.")
flags.DEFINE_integer("model_seed", 0, "Seed of the random weights.")
flags.DEFINE_float("matrix_std", 0.02, "Standard deviation of random matrices and embeddings.")
flags.DEFINE_float("scale_std", 0.0, "Standard deviation of random norm scales.")
flags.DEFINE_enum("weights_dtype", "bfloat16", ["bfloat16", "float32"], "Storage dtype of a written model folder.")
flags.DEFINE_integer("batch_size", 8, "Requests that may be live at once.")
flags.DEFINE_enum("activation_dtype", "bfloat16", ["float32", "bfloat16"], "Dtype of the activation.")
flags.DEFINE_integer("max_seq_len", 0, "Max sequence length; 0 means the model's max_position_embeddings.")
flags.DEFINE_integer("max_decode_steps", 256, "Max decode steps per request.")
flags.DEFINE_integer("page_size", 64, "Tokens per cache page.")
flags.DEFINE_integer("max_cache_tokens", 0, "Tokens the cache pool holds; 0 means batch_size * max_seq_len.")
flags.DEFINE_float("temperature", 1.0, "Temperature for sampling; 0 is greedy.")
flags.DEFINE_integer("top_k", -1, "Top-k for sampling; -1 is the whole vocabulary.")
flags.DEFINE_float("top_p", 1.0, "Top-p for sampling.")
flags.DEFINE_integer("intermediate_steps", 1, "Decode steps that run in a row without the host in between.")
flags.DEFINE_integer("max_num_issue_tokens", 0, "Token budget of one step; 0 means 2048.")
flags.DEFINE_integer("seed", 0, "Sampling seed; request i samples with seed + i.")
flags.DEFINE_bool("use_cuda_graphs", True, "Replay decode steps from CUDA graphs.")
flags.DEFINE_bool("logprobs", False, "Also print the log-probability of every output token.")
flags.DEFINE_string("prompt_ids", None, "Prompts as token ids: '1,2,3;4,5' (';' separates prompts).")
flags.DEFINE_string("prompt_file", None, "File with one prompt per line: token ids separated by spaces or commas.")
flags.DEFINE_string("prompt", None, "Prompts as text ('||' separates prompts); needs a vocabulary: --vocab_path, or "
                    "tokenizer.json / tokenizer.model in --ckpt_dir.")
flags.DEFINE_string("vocab_path", None, "Folder with tokenizer.json (and tokenizer_config.json), or a SentencePiece "
                    "model file (simply/serving/common_flags.py names vocabularies by --vocab_name).")


def _parse_ids(text: str) -> list[int]:
  return [int(t) for t in text.replace(",", " ").split()]


def _prompts() -> list[list[int]]:
  prompts: list[list[int]] = []
  if FLAGS.prompt_ids:
    prompts += [_parse_ids(p) for p in FLAGS.prompt_ids.split(";") if p.strip()]
  if FLAGS.prompt_file:
    with open(FLAGS.prompt_file) as f:
      prompts += [_parse_ids(line) for line in f if line.strip()]
  return prompts


def _named_config():
  from simply_b200.config import config_from_dict, preset, preset_dict
  if not FLAGS.config_overlay:
    return preset(FLAGS.experiment_config)
  text = FLAGS.config_overlay
  if os.path.exists(text):
    with open(text) as f:
      text = f.read()
  overlay = json.loads(text)
  if not isinstance(overlay, dict):
    raise app.UsageError("--config_overlay must be a JSON object")
  return config_from_dict({**preset_dict(FLAGS.experiment_config), **overlay})


def main(argv):
  del argv
  from simply_b200.config import EngineConfig
  from simply_b200.weights import write_model_folder

  if FLAGS.write_model_dir:
    if not FLAGS.experiment_config:
      raise app.UsageError("--write_model_dir needs --experiment_config")
    out = write_model_folder(_named_config(), FLAGS.model_seed, FLAGS.write_model_dir,
                             matrix_std=FLAGS.matrix_std, scale_std=FLAGS.scale_std, dtype=FLAGS.weights_dtype)
    print(json.dumps({"wrote": out}))
    return 0
  prompts = _prompts()
  if not prompts and not FLAGS.prompt:
    raise app.UsageError("give --prompt_ids, --prompt_file or --prompt")

  from simply_b200 import Engine, SamplingParams

  ec = EngineConfig(
      activation_dtype=FLAGS.activation_dtype, page_size=FLAGS.page_size, batch_size=FLAGS.batch_size,
      max_seq_len=FLAGS.max_seq_len, max_cache_tokens=FLAGS.max_cache_tokens,
      max_num_issue_tokens=FLAGS.max_num_issue_tokens, intermediate_steps=FLAGS.intermediate_steps,
      use_cuda_graphs=FLAGS.use_cuda_graphs)
  if FLAGS.ckpt_dir:
    engine = Engine.from_folder(FLAGS.ckpt_dir, ec)
  elif FLAGS.experiment_config and FLAGS.random_weights:
    engine = Engine.from_config(_named_config(), FLAGS.model_seed, ec,
                                matrix_std=FLAGS.matrix_std, scale_std=FLAGS.scale_std)
  else:
    raise app.UsageError("give --ckpt_dir, or --experiment_config with --random_weights")
  if FLAGS.prompt:
    from simply_b200.text import SentencePieceVocab, TextProcessor, load_vocab
    where = FLAGS.vocab_path or FLAGS.ckpt_dir
    if not where:
      raise app.UsageError("--prompt needs --vocab_path (or a model folder that holds a tokenizer)")
    vocab = SentencePieceVocab(where) if os.path.isfile(where) else load_vocab(where)
    processor = TextProcessor(vocab)
    texts = [t for t in FLAGS.prompt.split("||") if t.strip()]
    sp = SamplingParams(temperature=FLAGS.temperature, top_k=FLAGS.top_k, top_p=FLAGS.top_p,
                        max_decode_steps=FLAGS.max_decode_steps, seed=FLAGS.seed, logprobs=FLAGS.logprobs)
    for text, (answer, r) in zip(texts, engine.generate_text(texts, sp, processor=processor)):
      print(json.dumps({"request_id": r.request_id, "prompt": text, "text": answer,
                        "output_token_ids": r.output_token_ids, "finish_reason": r.finish_reason}))
    if not prompts:
      return 0
  params = [SamplingParams(temperature=FLAGS.temperature, top_k=FLAGS.top_k, top_p=FLAGS.top_p,
                           max_decode_steps=FLAGS.max_decode_steps, seed=FLAGS.seed + i, logprobs=FLAGS.logprobs)
            for i in range(len(prompts))]
  for r in engine.generate(prompts, params):
    line = {"request_id": r.request_id, "input_token_ids": r.input_token_ids,
            "output_token_ids": r.output_token_ids, "finish_reason": r.finish_reason,
            "is_truncated": r.is_truncated}
    if FLAGS.logprobs:
      line["output_token_logprobs"] = r.output_token_logprobs
    print(json.dumps(line))
  return 0


if __name__ == "__main__":
  app.run(main)
