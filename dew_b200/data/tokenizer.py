"""``ByteTokenizer``: UTF-8 bytes plus a few specials; needs no vocabulary file (reference: src/dew/data ByteTokenizer)."""
from __future__ import annotations

from typing import Iterable, List, Sequence


class ByteTokenizer:
    pad_id, bos_id, eos_id = 256, 257, 258
    vocab_size = 259

    def encode(self, text: str, bos: bool = False, eos: bool = False) -> List[int]:
        ids = list(text.encode("utf-8"))
        return ([self.bos_id] if bos else []) + ids + ([self.eos_id] if eos else [])

    def decode(self, ids: Iterable[int]) -> str:
        return bytes(i for i in ids if 0 <= int(i) < 256).decode("utf-8", errors="replace")

    def __call__(self, texts: Sequence[str], **kw):
        return [self.encode(t, **kw) for t in texts]
