"""Vocabularies, and the text processor that sits between text and the engine's token ids.

The engine itself speaks token ids.  This module is the optional step before and after it, after
the reference's `SimplyVocab` classes (simply/utils/tokenization.py:32-190: `encode`, `decode`,
`bos_id`, `eos_id`, `pad_id`; a whitespace test vocabulary :66-89, SentencePiece :91-140, the
`tokenizers` package's tokenizer.json :143-190) and its `BasicTextInputProcessor`
(simply/utils/sampling_lib.py:323-377: the bos id in front of the encoded text, the eos ids end a
request, a leading bos is dropped when decoding).

Vocabularies are registered by kind, like every other pluggable thing (simply_b200/registry.py);
`load_vocab(model_dir)` picks the kind by the files a model folder holds: `tokenizer.json` (with
`tokenizer_config.json` naming the special tokens) or `tokenizer.model`.  The tokenizer packages
are imported only when such a file is opened.
"""

from __future__ import annotations

import json
import os
from typing import Any, Sequence

from simply_b200.registry import Registry

VOCABS: Registry[Any] = Registry("vocab")


class Vocab:
  """Text <-> token ids, with the ids of the special tokens (None where the vocabulary has none)."""

  bos_id: int | None = None
  eos_id: int | None = None
  pad_id: int | None = None

  def encode(self, text: str) -> list[int]:
    raise NotImplementedError

  def decode(self, token_ids: Sequence[int]) -> str:
    raise NotImplementedError


@VOCABS.register("whitespace")
class WhitespaceVocab(Vocab):
  """Words separated by spaces; ids in the order given, after pad, bos, eos and unk (tests)."""

  def __init__(self, words: Sequence[str]):
    self.pad_id, self.bos_id, self.eos_id, self.unk_id = 0, 1, 2, 3
    self._words = ["<pad>", "<bos>", "<eos>", "<unk>", *words]
    self._ids = {w: i for i, w in enumerate(self._words)}

  def encode(self, text: str) -> list[int]:
    return [self._ids.get(w, self.unk_id) for w in text.split()]

  def decode(self, token_ids: Sequence[int]) -> str:
    return " ".join(self._words[i] if 0 <= i < len(self._words) else "<unk>" for i in token_ids)


@VOCABS.register("sentencepiece")
class SentencePieceVocab(Vocab):
  """A SentencePiece model file (`tokenizer.model`)."""

  def __init__(self, path: str):
    import sentencepiece

    self._sp = sentencepiece.SentencePieceProcessor()
    with open(path, "rb") as f:
      self._sp.LoadFromSerializedProto(f.read())

    def known(i: int) -> int | None:
      return i if i >= 0 else None

    self.bos_id, self.eos_id, self.pad_id = known(self._sp.bos_id()), known(self._sp.eos_id()), known(self._sp.pad_id())

  def encode(self, text: str) -> list[int]:
    return list(self._sp.EncodeAsIds(text))

  def decode(self, token_ids: Sequence[int]) -> str:
    return self._sp.DecodeIds(list(token_ids))


@VOCABS.register("huggingface")
class HuggingFaceVocab(Vocab):
  """A `tokenizer.json` of the `tokenizers` package; `tokenizer_config.json` beside it names the
  special tokens (`bos_token`, `eos_token`, `pad_token`: a string, or an object with `content`)."""

  def __init__(self, folder: str):
    import tokenizers

    self._tokenizer = tokenizers.Tokenizer.from_file(os.path.join(folder, "tokenizer.json"))
    config = {}
    path = os.path.join(folder, "tokenizer_config.json")
    if os.path.isfile(path):
      with open(path) as f:
        config = json.load(f)

    def special(name: str) -> int | None:
      token = config.get(name)
      if isinstance(token, dict):
        token = token.get("content")
      return self._tokenizer.token_to_id(token) if isinstance(token, str) else None

    self.bos_id, self.eos_id, self.pad_id = special("bos_token"), special("eos_token"), special("pad_token")

  def encode(self, text: str) -> list[int]:
    return list(self._tokenizer.encode(text, add_special_tokens=False).ids)

  def decode(self, token_ids: Sequence[int]) -> str:
    return self._tokenizer.decode(list(token_ids), skip_special_tokens=False)


def load_vocab(folder: str) -> Vocab:
  """The vocabulary a model folder brings: tokenizer.json, else tokenizer.model."""
  if os.path.isfile(os.path.join(folder, "tokenizer.json")):
    return HuggingFaceVocab(folder)
  if os.path.isfile(os.path.join(folder, "tokenizer.model")):
    return SentencePieceVocab(os.path.join(folder, "tokenizer.model"))
  raise FileNotFoundError(f"{folder!r} holds neither tokenizer.json nor tokenizer.model")


class TextProcessor:
  """Prompts to token ids (bos first) and generated ids back to text.

  eos_ids: the vocabulary's eos id plus `extra_eos_ids` and the ids of `extra_eos_tokens`, each of
  which must encode to a single token (simply/utils/sampling_lib.py:327-345)."""

  def __init__(self, vocab: Vocab, *, bos_id_override: int | None = None, extra_eos_ids: Sequence[int] = (),
               extra_eos_tokens: Sequence[str] = ()):
    self.vocab = vocab
    self.bos_id = bos_id_override if bos_id_override is not None else vocab.bos_id
    eos = [] if vocab.eos_id is None else [vocab.eos_id]
    eos += [int(i) for i in extra_eos_ids]
    for token in extra_eos_tokens:
      ids = vocab.encode(token)
      if len(ids) != 1:
        raise ValueError(f"eos token {token!r} encodes to {len(ids)} tokens; it must be a single token of the vocabulary")
      eos.append(ids[0])
    self.eos_ids = tuple(sorted(set(eos)))

  def encode(self, text: str, max_input_len: int | None = None) -> list[int]:
    tokens = ([] if self.bos_id is None else [self.bos_id]) + self.vocab.encode(text)
    return tokens[-max_input_len:] if max_input_len is not None else tokens

  def decode(self, token_ids: Sequence[int]) -> str:
    ids = list(token_ids)
    if ids and ids[0] == self.bos_id:
      ids = ids[1:]
    return self.vocab.decode(ids)
