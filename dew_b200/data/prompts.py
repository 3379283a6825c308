"""Prompts for online RL: fixed-width rows with their reward context.

``Prompts`` reads a parquet file, a JSON-lines file or in-memory rows in the common RL-data layout (``prompt`` - chat messages, a string
or token ids; ``data_source``; ``reward_model.ground_truth`` or ``ground_truth``; ``extra_info``).  Each row becomes a left-padded
``prompt [max_prompt_len]`` of ids with its ``prompt_length``, and the reward columns as fixed-width UTF-8 byte arrays, so every
leaf is a tensor that survives batching and a device transfer; ``decode_column`` reads them back.  A prompt longer than the window
keeps its tail (the question usually ends a prompt).  Messages are rendered with the chat template and a generation prompt.

Reference: src/dew/data/prompts.py (``Prompts``: left-padded prompts with ``data_source`` / ``ground_truth`` / ``extra_info``).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Mapping, Optional, Sequence, Union

import numpy as np

from .dataset import Dataset

COLUMNS = ("data_source", "ground_truth", "extra_info")


def encode_column(value: Any, width: int) -> np.ndarray:
    text = value if isinstance(value, str) else ("" if value is None else json.dumps(value, sort_keys=True))
    data = text.encode("utf-8")[:width]
    out = np.zeros(width, dtype=np.uint8)
    out[: len(data)] = np.frombuffer(data, dtype=np.uint8)
    return out


def decode_column(row) -> str:
    data = bytes(np.asarray(row, dtype=np.uint8).tolist())
    return data.rstrip(b"\x00").decode("utf-8", errors="ignore")


class Prompts(Dataset):
    def __init__(self, source: Union[str, Sequence[Mapping[str, Any]]], tokenizer, max_prompt_len: int = 512, pad_id: int = 0, column_width: int = 256,
                 template=None):
        if isinstance(source, (str, os.PathLike)):
            path = str(source)
            if path.endswith(".parquet"):
                import pyarrow.parquet as pq
                rows = pq.read_table(path).to_pylist()
            else:
                with open(path) as f:
                    rows = [json.loads(l) for l in f if l.strip()]
        else:
            rows = list(source)
        self._source, self.tokenizer, self.max_prompt_len, self.pad_id, self.column_width, self.template = rows, tokenizer, max_prompt_len, pad_id, column_width, template
        super().__init__(records=None, length=len(rows))

    def _ids(self, prompt) -> List[int]:
        if isinstance(prompt, str):
            return list(self.tokenizer.encode(prompt))
        if isinstance(prompt, (list, tuple)) and prompt and isinstance(prompt[0], Mapping):
            from .chat import render_prompt
            return render_prompt(self.tokenizer, list(prompt), self.template).tolist()
        return [int(t) for t in prompt]

    def _get(self, i: int) -> Dict[str, np.ndarray]:
        row = self._source[i]
        ids = self._ids(row["prompt"])[-self.max_prompt_len:]                # a prompt longer than the window keeps its tail
        padded = np.full(self.max_prompt_len, self.pad_id, dtype=np.int64)
        if ids:
            padded[-len(ids):] = ids                                          # left-padded: generation continues at the right edge
        truth = row.get("ground_truth")
        if truth is None and isinstance(row.get("reward_model"), Mapping):
            truth = row["reward_model"].get("ground_truth")
        out = {"prompt": padded, "prompt_length": np.int64(len(ids))}
        for name, value in (("data_source", row.get("data_source")), ("ground_truth", truth), ("extra_info", row.get("extra_info"))):
            out[name] = encode_column(value, self.column_width)
        return out
