"""A self-contained reader / writer for the safetensors container (8-byte little-endian header length, JSON header,
raw little-endian tensor bytes), so checkpoints need no package beyond PyTorch."""
from __future__ import annotations

import json
import os
import struct
from pathlib import Path
from typing import Dict, Mapping, Optional

import numpy as np
import torch

_DT = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.float64: "F64", torch.int64: "I64",
       torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8", torch.bool: "BOOL",
       torch.float8_e4m3fn: "F8_E4M3", torch.float8_e5m2: "F8_E5M2"}
_RT = {v: k for k, v in _DT.items()}


def _bytes(t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous()
    if t.numel() == 0:
        return b""
    return t.reshape(-1).view(torch.uint8).numpy().tobytes()


def save_file(tensors: Mapping[str, torch.Tensor], path: os.PathLike, metadata: Optional[Dict[str, str]] = None) -> None:
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name]
        b = _bytes(t)
        header[name] = {"dtype": _DT[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(b)]}
        offset += len(b)
        blobs.append(b)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = Path(str(path) + ".tmp")
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def read_header(path: os.PathLike):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        return json.loads(f.read(n)), 8 + n


def load_file(path: os.PathLike, device="cpu", names=None) -> Dict[str, torch.Tensor]:
    header, base = read_header(path)
    out: Dict[str, torch.Tensor] = {}
    data = np.memmap(path, dtype=np.uint8, mode="r", offset=base) if os.path.getsize(path) > base else np.zeros(0, np.uint8)
    for name, info in header.items():
        if name == "__metadata__" or (names is not None and name not in names):
            continue
        lo, hi = info["data_offsets"]
        dt = _RT[info["dtype"]]
        raw = torch.from_numpy(np.array(data[lo:hi], copy=True))
        t = raw.view(dt).reshape(info["shape"]) if hi > lo else torch.empty(info["shape"], dtype=dt)
        out[name] = t.to(device)
    return out


def load_metadata(path: os.PathLike) -> Dict[str, str]:
    header, _ = read_header(path)
    return header.get("__metadata__", {})
