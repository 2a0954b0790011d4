"""Tokenizer seam for text sources: ``gpt2`` / ``tiktoken:ENC`` (tiktoken), ``hf:NAME`` (transformers) and
``bytes`` (UTF-8 bytes + one end-of-text id; needs no package, used by tests and air-gapped boxes).
``encode`` is deterministic and never truncates; the identity lands in run metadata.
Contract parity: reference ``src/dataflow_training/data/tokenizers.py:28-85``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any


@dataclass
class Tokenizer:
    backend: str
    name: str
    vocab_size: int
    eot_id: int | None
    _impl: Any = None

    def encode(self, text: str) -> list[int]:
        if self.backend == "bytes":
            return list(text.encode("utf-8"))
        if self.backend == "tiktoken":
            return self._impl.encode_ordinary(text)
        return self._impl.encode(text, add_special_tokens=False)

    def describe(self) -> dict:
        return {"backend": self.backend, "name": self.name, "vocab_size": self.vocab_size, "eot_id": self.eot_id}


def resolve_tokenizer(spec: str) -> Tokenizer:
    if spec == "bytes":
        return Tokenizer("bytes", "utf8", 257, 256)
    if spec == "gpt2" or spec.startswith("tiktoken:"):
        enc_name = "gpt2" if spec == "gpt2" else spec.split(":", 1)[1]
        try:
            import tiktoken
        except ImportError as e:       # noqa: F841
            raise RuntimeError(f"tokenizer {spec!r} needs the tiktoken package (not installed here); "
                               "use tokenizer=bytes or hf:NAME") from None
        enc = tiktoken.get_encoding(enc_name)
        return Tokenizer("tiktoken", enc_name, enc.n_vocab, enc.eot_token, enc)
    if spec.startswith("hf:"):
        name = spec[3:]
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(name)
        return Tokenizer("hf", name, len(tok), tok.eos_token_id, tok)
    raise KeyError(f"unknown tokenizer {spec!r} (bytes | gpt2 | tiktoken:ENC | hf:NAME)")
