"""Pipeline presets (reference: src/dew/data presets ``images / lm / token_windows / sft / preferences / prompts``)."""
from __future__ import annotations

from typing import Any, Callable, List, Mapping, Optional, Sequence

import numpy as np
import torch

from .dataset import Dataset, Memory


def images(ds: Dataset, *, batch: int, key: str = "image", out: str = "sample", size: Optional[int] = None) -> Dataset:
    """uint8 / float NHWC images -> ``{'sample': float32 in [-1, 1]}`` batches."""
    def prep(r):
        x = torch.as_tensor(np.asarray(r[key]))
        if x.dtype == torch.uint8:
            x = x.float() / 127.5 - 1.0
        rest = {k: v for k, v in r.items() if k != key}
        return {out: x.float(), **rest}
    return ds.map(prep).batched(batch)


def pack_documents(docs: Sequence[Sequence[int]], seq_len: int, pad_id: int, eos_id: Optional[int] = None):
    """Greedy first-fit packing into rows of ``seq_len + 1`` tokens with segment ids (0 = padding)."""
    rows: List[List[int]] = []
    segs: List[List[int]] = []
    cur, cur_seg, seg = [], [], 1
    L = seq_len + 1
    for d in docs:
        d = list(d) + ([eos_id] if eos_id is not None else [])
        while d:
            space = L - len(cur)
            take = d[:space]
            cur += take
            cur_seg += [seg] * len(take)
            d = d[space:]
            if len(cur) == L:
                rows.append(cur); segs.append(cur_seg)
                cur, cur_seg = [], []
            seg += 1
    if cur:
        pad = L - len(cur)
        rows.append(cur + [pad_id] * pad)
        segs.append(cur_seg + [0] * pad)
    return np.asarray(rows, dtype=np.int64), np.asarray(segs, dtype=np.int32)


def lm(ds: Dataset, tokenizer, *, seq_len: int, batch: int, pack: bool = True, text_key: str = "text") -> Dataset:
    """Text records -> ``{'tokens': [B, seq_len + 1]}`` (inputs are ``[:, :-1]``, targets ``[:, 1:]``)."""
    docs = []
    for i in range(len(ds)):
        r = ds._get(i)
        text = r[text_key] if isinstance(r, Mapping) else r
        docs.append(tokenizer.encode(text))
    pad = getattr(tokenizer, "pad_id", 0)
    eos = getattr(tokenizer, "eos_id", None)
    if pack:
        rows, segs = pack_documents(docs, seq_len, pad, eos)
    else:
        rows = np.full((len(docs), seq_len + 1), pad, dtype=np.int64)
        segs = np.zeros((len(docs), seq_len + 1), dtype=np.int32)
        for i, d in enumerate(docs):
            d = (d + ([eos] if eos is not None else []))[: seq_len + 1]
            rows[i, :len(d)] = d
            segs[i, :len(d)] = 1
    out = Memory({"tokens": torch.from_numpy(rows), "segments": torch.from_numpy(segs)})
    out._shuffle_seed, out._repeat = ds._shuffle_seed, ds._repeat
    out = out.batched(batch)
    out.seq_len = seq_len
    return out


def token_windows(ds, *, seq_len: int, batch: int) -> Dataset:
    """Fixed windows of ``seq_len + 1`` tokens from flat token files."""
    out = ds.set_window(seq_len + 1).batched(batch)
    out.seq_len = seq_len
    return out


def sft(ds: Dataset, tokenizer, *, seq_len: int, batch: int, prompt_key: str = "prompt", response_key: str = "response") -> Dataset:
    """Prompt/response pairs -> tokens plus a loss mask that scores only the response."""
    pad = getattr(tokenizer, "pad_id", 0)

    def prep(r):
        p = tokenizer.encode(r[prompt_key])
        a = tokenizer.encode(r[response_key]) + [getattr(tokenizer, "eos_id", pad)]
        ids = (p + a)[: seq_len + 1]
        mask = ([0] * len(p) + [1] * len(a))[: seq_len + 1]
        n = len(ids)
        return {"tokens": torch.tensor(ids + [pad] * (seq_len + 1 - n)), "loss_mask": torch.tensor(mask + [0] * (seq_len + 1 - n))}
    out = ds.map(prep).batched(batch)
    out.seq_len = seq_len
    return out


def preferences(ds: Dataset, tokenizer, *, seq_len: int, batch: int) -> Dataset:
    """(prompt, chosen, rejected) -> two token rows and masks, for DPO."""
    pad = getattr(tokenizer, "pad_id", 0)

    def side(p, a):
        ids = (p + a)[: seq_len + 1]
        mask = ([0] * len(p) + [1] * len(a))[: seq_len + 1]
        n = len(ids)
        return torch.tensor(ids + [pad] * (seq_len + 1 - n)), torch.tensor(mask + [0] * (seq_len + 1 - n))

    def prep(r):
        p = tokenizer.encode(r["prompt"])
        c, cm = side(p, tokenizer.encode(r["chosen"]))
        j, jm = side(p, tokenizer.encode(r["rejected"]))
        return {"chosen": c, "chosen_mask": cm, "rejected": j, "rejected_mask": jm}
    out = ds.map(prep).batched(batch)
    out.seq_len = seq_len
    return out


def prompts(ds: Dataset, tokenizer, *, batch: int, max_len: int = 512) -> Dataset:
    def prep(r):
        text = r["prompt"] if isinstance(r, Mapping) else r
        return {"prompt_ids": tokenizer.encode(text)[:max_len], "prompt": text}
    return ds.map(prep).batched(batch)
