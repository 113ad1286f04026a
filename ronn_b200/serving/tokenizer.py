"""Tokenizers for the text endpoints of the HTTP front end.

The runtime itself works on token ids.  The chat endpoint of the continuous-batching design
(docs/new/RONN-Continuous-Batching-Branch-Prompt.md:377-395, ``/v1/chat/completions``) takes text, so the server
accepts any object with ``encode(str) -> List[int]`` and ``decode(List[int]) -> str``.  Two are provided:

* ``ByteTokenizer``: UTF-8 bytes as ids 0..255 (needs a vocabulary of at least 256); works with any random-init model
  and is what the tests use;
* ``SentencePieceTokenizer``: a ``.model`` file loaded with the ``sentencepiece`` package (Llama-family vocabularies;
  the Llama design names a BPE tokenizer, docs/new/RONN-Llama-Branch-Prompt.md:793-889).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence


class ByteTokenizer:
    """ids = UTF-8 bytes (+ ``offset``).  Ids outside the byte range decode to U+FFFD."""

    def __init__(self, vocab_size: int = 256, offset: int = 0):
        if vocab_size < offset + 256:
            raise ValueError(f"a byte tokenizer needs {offset + 256} vocabulary entries, the model has {vocab_size}")
        self.offset = offset
        self.vocab_size = vocab_size

    def encode(self, text: str) -> List[int]:
        return [b + self.offset for b in text.encode("utf-8")]

    def decode(self, ids: Sequence[int]) -> str:
        out = bytearray()
        for i in ids:
            j = int(i) - self.offset
            out += bytes([j]) if 0 <= j < 256 else "�".encode("utf-8")
        return out.decode("utf-8", errors="replace")


class SentencePieceTokenizer:
    def __init__(self, path: str):
        import sentencepiece as spm
        self.sp = spm.SentencePieceProcessor(model_file=path)
        self.vocab_size = self.sp.get_piece_size()

    def encode(self, text: str) -> List[int]:
        return list(self.sp.encode(text))

    def decode(self, ids: Sequence[int]) -> str:
        return self.sp.decode([int(i) for i in ids])


def load_tokenizer(spec: Optional[str], vocab_size: int):
    """``None`` / ``"bytes"`` -> ByteTokenizer when the vocabulary allows it (else None); a path -> SentencePiece."""
    if spec in (None, "", "bytes"):
        return ByteTokenizer(vocab_size) if vocab_size >= 256 else None
    return SentencePieceTokenizer(spec)


def render_chat(messages: Sequence[Dict[str, str]]) -> str:
    """Plain chat template: one ``role: content`` line per message and an open assistant line."""
    lines = [f"{m.get('role', 'user')}: {m.get('content', '')}" for m in messages]
    lines.append("assistant:")
    return "\n".join(lines)
