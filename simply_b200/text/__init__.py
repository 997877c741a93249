"""Text in, text out: vocabularies and the step from text to token ids and back."""

from simply_b200.text.vocab import (TextProcessor, Vocab, VOCABS, load_vocab, HuggingFaceVocab, SentencePieceVocab,
                                    WhitespaceVocab)

__all__ = ["HuggingFaceVocab", "SentencePieceVocab", "TextProcessor", "VOCABS", "Vocab", "WhitespaceVocab",
           "load_vocab"]
