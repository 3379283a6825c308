"""GGUF reader (and a minimal writer for tests): the single-file checkpoint format of llama.cpp.

Layout (little endian): magic ``GGUF``, version (3), tensor count, metadata count; metadata key-value pairs (typed:
integers, floats, bool, string, arrays); tensor infos (name, dims innermost first, ggml type, data offset); padding to the
alignment (``general.alignment``, default 32); tensor data.  Supported tensor types: F32, F16, BF16 and the block formats
Q8_0 (32 int8 + one fp16 scale) and Q4_0 (32 4-bit values + one fp16 scale), which are dequantised on load.

Reference: src/dew/interop (GGUF and quantised loads among the 55 files of the package).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Any, BinaryIO, Dict, List, Tuple

import numpy as np
import torch

MAGIC = b"GGUF"
F32, F16, Q4_0, Q8_0, BF16 = 0, 1, 2, 8, 30
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_STRING, _ARRAY = 8, 9
BLOCK = 32


@dataclass
class TensorInfo:
    name: str
    shape: Tuple[int, ...]       # outermost first (as torch sees it)
    ggml_type: int
    offset: int


def _read(f: BinaryIO, fmt: str):
    size = struct.calcsize(fmt)
    return struct.unpack(fmt, f.read(size))[0]


def _read_string(f: BinaryIO) -> str:
    n = _read(f, "<Q")
    return f.read(n).decode("utf-8")


def _read_value(f: BinaryIO, kind: int):
    if kind in _SCALARS:
        return _read(f, _SCALARS[kind])
    if kind == _STRING:
        return _read_string(f)
    if kind == _ARRAY:
        inner = _read(f, "<I")
        n = _read(f, "<Q")
        return [_read_value(f, inner) for _ in range(n)]
    raise ValueError(f"unknown GGUF metadata type {kind}")


def _nbytes(ggml_type: int, numel: int) -> int:
    if ggml_type == F32:
        return 4 * numel
    if ggml_type in (F16, BF16):
        return 2 * numel
    if ggml_type == Q8_0:
        return numel // BLOCK * (2 + BLOCK)
    if ggml_type == Q4_0:
        return numel // BLOCK * (2 + BLOCK // 2)
    raise ValueError(f"unsupported ggml tensor type {ggml_type}")


def dequantize(raw: bytes, ggml_type: int, shape: Tuple[int, ...]) -> torch.Tensor:
    numel = int(np.prod(shape)) if shape else 1
    if ggml_type == F32:
        return torch.from_numpy(np.frombuffer(raw, dtype="<f4", count=numel).copy()).reshape(shape)
    if ggml_type == F16:
        return torch.from_numpy(np.frombuffer(raw, dtype="<f2", count=numel).copy()).reshape(shape)
    if ggml_type == BF16:
        bits = torch.from_numpy(np.frombuffer(raw, dtype="<u2", count=numel).astype(np.int32))
        return (bits << 16).view(torch.float32).to(torch.bfloat16).reshape(shape)
    blocks = numel // BLOCK
    if ggml_type == Q8_0:
        rec = np.frombuffer(raw, dtype=np.dtype([("d", "<f2"), ("q", "i1", (BLOCK,))]), count=blocks)
        return torch.from_numpy((rec["d"].astype(np.float32)[:, None] * rec["q"].astype(np.float32)).reshape(shape))
    if ggml_type == Q4_0:
        rec = np.frombuffer(raw, dtype=np.dtype([("d", "<f2"), ("q", "u1", (BLOCK // 2,))]), count=blocks)
        lo = (rec["q"] & 0x0F).astype(np.float32) - 8.0      # the first 16 values of a block are the low nibbles
        hi = (rec["q"] >> 4).astype(np.float32) - 8.0
        vals = np.concatenate([lo, hi], 1) * rec["d"].astype(np.float32)[:, None]
        return torch.from_numpy(vals.reshape(shape))
    raise ValueError(f"unsupported ggml tensor type {ggml_type}")


def read(path: str, load_tensors: bool = True):
    """-> (metadata dict, {name: tensor}) (or the ``TensorInfo`` list when ``load_tensors`` is false)."""
    with open(path, "rb") as f:
        if f.read(4) != MAGIC:
            raise ValueError(f"{path} is not a GGUF file")
        version = _read(f, "<I")
        if version not in (2, 3):
            raise ValueError(f"GGUF version {version} is not supported")
        n_tensors, n_meta = _read(f, "<Q"), _read(f, "<Q")
        meta: Dict[str, Any] = {}
        for _ in range(n_meta):
            key = _read_string(f)
            meta[key] = _read_value(f, _read(f, "<I"))
        infos: List[TensorInfo] = []
        for _ in range(n_tensors):
            name = _read_string(f)
            nd = _read(f, "<I")
            dims = [_read(f, "<Q") for _ in range(nd)]
            infos.append(TensorInfo(name, tuple(reversed(dims)), _read(f, "<I"), _read(f, "<Q")))
        align = int(meta.get("general.alignment", 32))
        base = (f.tell() + align - 1) // align * align
        if not load_tensors:
            return meta, infos
        tensors = {}
        for info in infos:
            numel = int(np.prod(info.shape)) if info.shape else 1
            f.seek(base + info.offset)
            tensors[info.name] = dequantize(f.read(_nbytes(info.ggml_type, numel)), info.ggml_type, info.shape)
        return meta, tensors


def quantize_q8_0(t: torch.Tensor) -> bytes:
    x = t.float().reshape(-1, BLOCK).numpy()
    d = np.abs(x).max(1) / 127.0
    q = np.where(d[:, None] > 0, np.round(x / np.where(d[:, None] > 0, d[:, None], 1.0)), 0).astype(np.int8)
    rec = np.zeros(len(x), dtype=np.dtype([("d", "<f2"), ("q", "i1", (BLOCK,))]))
    rec["d"], rec["q"] = d.astype(np.float16), q
    return rec.tobytes()


def write(path: str, metadata: Dict[str, Any], tensors: Dict[str, torch.Tensor], quantize: Dict[str, int] = None, align: int = 32) -> None:
    """Writer for round-trip tests and small exports: F32 / F16 / BF16 / Q8_0 tensors, scalar / string / list metadata."""
    quantize = quantize or {}

    def w_string(b: bytearray, s: str):
        raw = s.encode("utf-8")
        b += struct.pack("<Q", len(raw)) + raw

    def w_value(b: bytearray, v):
        if isinstance(v, bool):
            b += struct.pack("<I", 7) + struct.pack("<?", v)
        elif isinstance(v, int):
            b += struct.pack("<I", 11) + struct.pack("<q", v)
        elif isinstance(v, float):
            b += struct.pack("<I", 6) + struct.pack("<f", v)
        elif isinstance(v, str):
            b += struct.pack("<I", _STRING)
            w_string(b, v)
        elif isinstance(v, (list, tuple)):
            inner = 8 if (v and isinstance(v[0], str)) else (6 if (v and isinstance(v[0], float)) else 11)
            b += struct.pack("<I", _ARRAY) + struct.pack("<I", inner) + struct.pack("<Q", len(v))
            for item in v:
                if inner == 8:
                    w_string(b, item)
                else:
                    b += struct.pack("<f" if inner == 6 else "<q", item)
        else:
            raise TypeError(f"cannot store {type(v)} in GGUF metadata")

    head = bytearray(MAGIC + struct.pack("<I", 3) + struct.pack("<Q", len(tensors)) + struct.pack("<Q", len(metadata) + 1))
    w_string(head, "general.alignment")
    head += struct.pack("<I", 4) + struct.pack("<I", align)
    for k, v in metadata.items():
        w_string(head, k)
        w_value(head, v)
    blobs, offset = [], 0
    for name, t in tensors.items():
        kind = quantize.get(name, {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[t.dtype])
        if kind == Q8_0:
            raw = quantize_q8_0(t)
        elif kind == BF16:
            raw = t.contiguous().view(torch.int16).numpy().tobytes()
        else:
            raw = t.contiguous().numpy().tobytes()
        w_string(head, name)
        head += struct.pack("<I", t.dim())
        for dim in reversed(t.shape):
            head += struct.pack("<Q", dim)
        head += struct.pack("<I", kind) + struct.pack("<Q", offset)
        blobs.append(raw)
        offset += (len(raw) + align - 1) // align * align
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\x00" * ((len(head) + align - 1) // align * align - len(head)))
        for raw in blobs:
            f.write(raw)
            f.write(b"\x00" * ((len(raw) + align - 1) // align * align - len(raw)))
