"""A published checkpoint directory: ``config.json``, ``generation_config.json``, one ``model.safetensors`` or shards named
by ``model.safetensors.index.json``.  ``Release`` is a read-only mapping from tensor name to tensor that opens the shard
a name lives in only when the name is read (so a loader that walks layer by layer never holds more than it copies), and
that de-quantises the stored forms releases ship: fp8 weights with ``*_scale_inv`` block scales (128 x 128 blocks unless
the config says otherwise) or a per-tensor ``*_scale``.  ``save_release`` writes the same layout with a size limit per
shard.

Reference: src/dew/interop/pretrained.py, safetensors_io.py, streaming.py (shard-at-a-time loads), quantized_loads.py /
codecs.py (stored quantised formats), generation_config.py, release_record.py.
"""
from __future__ import annotations

import json
import os
from collections.abc import Mapping as _Mapping
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Dict, Iterator, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from ..checkpoints import tensors as TS

INDEX = "model.safetensors.index.json"


@dataclass
class GenerationConfig:
    """The sampling defaults a release ships beside its weights."""
    max_new_tokens: Optional[int] = None
    do_sample: bool = False
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    eos_token_id: Any = None                       # one id or a list of ids
    bos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None

    @classmethod
    def read(cls, directory: os.PathLike) -> "GenerationConfig":
        p = Path(directory) / "generation_config.json"
        if not p.exists():
            return cls()
        raw = json.loads(p.read_text())
        known = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in raw.items() if k in known})

    def write(self, directory: os.PathLike) -> None:
        (Path(directory) / "generation_config.json").write_text(json.dumps({k: v for k, v in asdict(self).items() if v is not None}, indent=1))

    def stop_ids(self) -> Tuple[int, ...]:
        e = self.eos_token_id
        return () if e is None else (tuple(int(x) for x in e) if isinstance(e, (list, tuple)) else (int(e),))


def dequantize_blocks(q: torch.Tensor, scale_inv: torch.Tensor, block: Sequence[int] = (128, 128), dtype=torch.bfloat16) -> torch.Tensor:
    """``q [out, in]`` (fp8 or int8) times one scale per ``block[0] x block[1]`` tile (``scale_inv [ceil(out/b0), ceil(in/b1)]``)."""
    out, inn = q.shape
    b0, b1 = int(block[0]), int(block[1])
    s = scale_inv.float().repeat_interleave(b0, 0)[:out].repeat_interleave(b1, 1)[:, :inn]
    return (q.float() * s).to(dtype)


def quantize_blocks(w: torch.Tensor, block: Sequence[int] = (128, 128)) -> Tuple[torch.Tensor, torch.Tensor]:
    """The inverse layout: e4m3 values and the fp32 ``scale_inv`` per tile (amax / 448)."""
    out, inn = w.shape
    b0, b1 = int(block[0]), int(block[1])
    po, pi = (-out) % b0, (-inn) % b1
    wf = torch.nn.functional.pad(w.float(), (0, pi, 0, po))
    tiles = wf.reshape((out + po) // b0, b0, (inn + pi) // b1, b1)
    scale = tiles.abs().amax((1, 3)).clamp_min(1e-12) / 448.0
    q = (tiles / scale[:, None, :, None]).reshape(out + po, inn + pi)[:out, :inn].to(torch.float8_e4m3fn)
    return q, scale


class Release(_Mapping):
    """Tensors of a checkpoint directory by name, read on demand."""

    def __init__(self, directory: os.PathLike, dequantize: bool = True, dtype=torch.bfloat16):
        self.dir = Path(directory)
        self.config: Dict[str, Any] = json.loads((self.dir / "config.json").read_text()) if (self.dir / "config.json").exists() else {}
        self.dequantize, self.dtype = dequantize, dtype
        self._where: Dict[str, str] = {}
        idx = self.dir / INDEX
        if idx.exists():
            self._where = dict(json.loads(idx.read_text())["weight_map"])
        else:
            for f in sorted(self.dir.glob("*.safetensors")):
                header, _ = TS.read_header(f)
                for name in header:
                    if name != "__metadata__":
                        self._where[name] = f.name
        if not self._where:
            raise FileNotFoundError(f"no safetensors files under {self.dir}")
        self._headers: Dict[str, Tuple[dict, int]] = {}
        qc = self.config.get("quantization_config") or {}
        self.block = tuple(qc.get("weight_block_size") or (128, 128))
        self.opened: List[str] = []                       # shard files in the order they were first opened

    # scales are consumed by their weight: they are not names of the mapping when de-quantising
    def _is_scale(self, name: str) -> bool:
        return self.dequantize and (name.endswith("_scale_inv") or name.endswith(".weight_scale")) and \
            (name.rsplit("_scale", 1)[0] in self._where)

    def __iter__(self) -> Iterator[str]:
        return (k for k in self._where if not self._is_scale(k))

    def __len__(self) -> int:
        return sum(1 for _ in self)

    def __contains__(self, name: object) -> bool:
        return name in self._where and not self._is_scale(str(name))

    def _raw(self, name: str) -> torch.Tensor:
        fname = self._where[name]
        if fname not in self._headers:
            self._headers[fname] = TS.read_header(self.dir / fname)
            self.opened.append(fname)
        header, base = self._headers[fname]
        info = header[name]
        lo, hi = info["data_offsets"]
        dt = TS._RT[info["dtype"]]
        if hi == lo:
            return torch.empty(info["shape"], dtype=dt)
        raw = np.fromfile(self.dir / fname, dtype=np.uint8, count=hi - lo, offset=base + lo)
        return torch.from_numpy(raw).view(dt).reshape(info["shape"])

    def __getitem__(self, name: str) -> torch.Tensor:
        if name not in self._where:
            raise KeyError(name)
        t = self._raw(name)
        if not self.dequantize or t.dtype not in (torch.float8_e4m3fn, torch.float8_e5m2, torch.int8):
            return t
        if name + "_scale_inv" in self._where:
            return dequantize_blocks(t, self._raw(name + "_scale_inv"), self.block, self.dtype)
        if name + "_scale" in self._where:
            s = self._raw(name + "_scale").float()
            return (t.float() * (s if s.dim() == 0 or s.numel() == 1 else s.reshape(-1, 1))).to(self.dtype)
        return t

    def bytes_on_disk(self) -> int:
        return sum((self.dir / f).stat().st_size for f in set(self._where.values()))


def save_release(tensors: Mapping[str, torch.Tensor], config: Mapping[str, Any], directory: os.PathLike,
                 max_shard_bytes: int = 5 << 30, generation: Optional[GenerationConfig] = None,
                 fp8_blocks: Optional[Sequence[int]] = None, skip_fp8: Sequence[str] = ("embed", "norm", "lm_head", "gate.weight")) -> List[str]:
    """Write ``tensors`` as one file, or as shards of at most ``max_shard_bytes`` with an index, beside ``config.json``.
    ``fp8_blocks=(128, 128)`` stores every 2-D weight not named in ``skip_fp8`` as e4m3 with block scales (and says so in the
    config's ``quantization_config``).  Returns the file names written."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    config = dict(config)
    stored: Dict[str, torch.Tensor] = {}
    for k, t in tensors.items():
        if fp8_blocks and t.dim() == 2 and k.endswith(".weight") and not any(s in k for s in skip_fp8):
            q, s = quantize_blocks(t, fp8_blocks)
            stored[k], stored[k + "_scale_inv"] = q, s
        else:
            stored[k] = t
    if fp8_blocks:
        config["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": list(fp8_blocks), "activation_scheme": "dynamic"}
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    for k in sorted(stored):
        n = stored[k].numel() * stored[k].element_size()
        if shards[-1] and size + n > max_shard_bytes:
            shards.append({})
            size = 0
        shards[-1][k] = stored[k]
        size += n
    (d / "config.json").write_text(json.dumps(config, indent=1))
    if generation is not None:
        generation.write(d)
    if len(shards) == 1:
        TS.save_file(shards[0], d / "model.safetensors", metadata={"format": "pt"})
        return ["model.safetensors"]
    names, where = [], {}
    for i, shard in enumerate(shards, start=1):
        fname = f"model-{i:05d}-of-{len(shards):05d}.safetensors"
        TS.save_file(shard, d / fname, metadata={"format": "pt"})
        names.append(fname)
        where.update({k: fname for k in shard})
    total = sum(t.numel() * t.element_size() for t in stored.values())
    (d / INDEX).write_text(json.dumps({"metadata": {"total_size": total}, "weight_map": where}, indent=1))
    return names
