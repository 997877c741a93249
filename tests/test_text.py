"""Text in, text out: vocabularies and the text processor (simply/utils/tokenization.py,
simply/utils/sampling_lib.py:323-377), and `Engine.generate_text` on the CPU kernel table."""

import json

import numpy as np
import pytest
import torch

from simply_b200 import Engine, EngineConfig, SamplingParams
from simply_b200.text import TextProcessor, VOCABS, WhitespaceVocab, load_vocab
from tests.plain.gemma2_plain import PlainGemma2
from tests.reference_ops import ReferenceOps
from tests.tiny_models import write_tiny

WORDS = [f"w{i}" for i in range(200)]


def test_text_processor_puts_bos_first_and_knows_the_eos_ids():
  vocab = WhitespaceVocab(WORDS)
  p = TextProcessor(vocab, extra_eos_ids=[9], extra_eos_tokens=["w7"])
  assert p.encode("w0 w5 nope") == [1, 4, 9, 3]  # bos, two words, unk
  assert p.eos_ids == (2, 9, 11)
  assert p.decode([1, 4, 9]) == "w0 w5" and p.decode([4, 9]) == "w0 w5"  # a leading bos is dropped
  assert p.encode("w0 w1 w2 w3", max_input_len=2) == [6, 7]  # the last tokens are kept
  with pytest.raises(ValueError, match="single token"):
    TextProcessor(vocab, extra_eos_tokens=["w1 w2"])
  assert TextProcessor(vocab, bos_id_override=5).encode("w0")[0] == 5
  assert VOCABS.get("whitespace") is WhitespaceVocab and "huggingface" in VOCABS and "sentencepiece" in VOCABS


def test_a_tokenizer_json_in_the_model_folder(tmp_path):
  tokenizers = pytest.importorskip("tokenizers")
  from tokenizers import models, pre_tokenizers
  vocab = {"<pad>": 0, "<bos>": 1, "<eos>": 2, "<unk>": 3, **{w: 4 + i for i, w in enumerate(WORDS)}}
  tok = tokenizers.Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
  tok.pre_tokenizer = pre_tokenizers.Whitespace()
  tok.save(str(tmp_path / "tokenizer.json"))
  (tmp_path / "tokenizer_config.json").write_text(json.dumps(
      {"bos_token": "<bos>", "eos_token": {"content": "<eos>"}, "pad_token": None}))
  v = load_vocab(str(tmp_path))
  assert (v.bos_id, v.eos_id, v.pad_id) == (1, 2, None)
  assert v.encode("w3 w10") == [7, 14] and v.decode([7, 14]) == "w3 w10"
  with pytest.raises(FileNotFoundError):
    load_vocab(str(tmp_path / "nowhere"))


def test_generate_text_on_the_cpu_kernel_table(tmp_path):
  folder = write_tiny("a", tmp_path)  # vocabulary of 256 ids: 4 special + 200 words fit
  plain = PlainGemma2(folder)
  eng = Engine.from_folder(folder, EngineConfig(activation_dtype="float32", page_size=4, batch_size=2, max_seq_len=64),
                           ops=ReferenceOps(torch.float32))
  processor = TextProcessor(WhitespaceVocab(WORDS))
  prompts = ["w1 w2 w3", "w9"]
  ids = [processor.encode(p) for p in prompts]
  assert ids[0] == [1, 5, 6, 7]
  # no stop token is hit in six steps here: the text is the decoded ids
  want = [plain.greedy(i, 6) for i in ids]
  got = eng.generate_text(prompts, SamplingParams(temperature=0.0, max_decode_steps=6, stop_token_ids=()),
                          processor=processor)
  assert [r.output_token_ids for _, r in got] == want
  assert [t for t, _ in got] == [processor.decode(w) for w in want]
  # with the processor's eos ids: a request ends on one of them and the text leaves it out
  stop = want[0][2]
  p2 = TextProcessor(WhitespaceVocab(WORDS), extra_eos_ids=[stop])
  text, r = eng.generate_text(prompts[:1], SamplingParams(temperature=0.0, max_decode_steps=6), processor=p2)[0]
  first = want[0].index(stop)
  assert r.finish_reason == "eos" and r.output_token_ids == want[0][:first + 1]
  assert text == p2.decode(want[0][:first])
