"""Tokenizers: the checkpoint's ``tokenizer.json`` (HF tokenizers) or a byte fallback.

The byte fallback maps UTF-8 bytes to ids 3..258 (0 pad, 1 bos, 2 eos), which is what the hermetic
CPU tests and random-weight benches use.  Incremental detokenisation holds back bytes until
they form complete UTF-8 so streamed deltas never contain a broken code point (reference:
crates/plowrt/src/text/{tokenizer,detok}.rs).
"""
from __future__ import annotations

from pathlib import Path


class ByteTokenizer:
    bos_id, eos_id, pad_id = 1, 2, 0
    vocab_size = 259

    def encode(self, text: str, add_bos: bool = False) -> list:
        ids = [b + 3 for b in text.encode("utf-8")]
        return ([self.bos_id] if add_bos else []) + ids

    def decode(self, ids) -> str:
        return bytes(i - 3 for i in ids if 3 <= i < 259).decode("utf-8", errors="replace")

    def decode_bytes(self, ids) -> bytes:
        return bytes(i - 3 for i in ids if 3 <= i < 259)


class HfTokenizer:
    def __init__(self, path):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(str(path))
        self.vocab_size = self.tk.get_vocab_size()
        self.bos_id = self.eos_id = None

    def encode(self, text: str, add_bos: bool = False) -> list:
        return self.tk.encode(text, add_special_tokens=add_bos).ids

    def decode(self, ids) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=True)


def load_tokenizer(assets_dir):
    p = Path(assets_dir) / "tokenizer.json"
    return HfTokenizer(p) if p.exists() else ByteTokenizer()


class IncrementalDetok:
    """Streams text deltas; never emits a partial UTF-8 sequence or a half-merged token."""

    def __init__(self, tok):
        self.tok = tok
        self.ids: list = []
        self.emitted = ""

    def push(self, token_id: int) -> str:
        self.ids.append(token_id)
        text = self.tok.decode(self.ids)
        if text.endswith("�"):
            return ""
        delta = text[len(self.emitted):]
        self.emitted = text
        return delta

    def flush(self) -> str:
        text = self.tok.decode(self.ids)
        delta = text[len(self.emitted):]
        self.emitted = text
        return delta
