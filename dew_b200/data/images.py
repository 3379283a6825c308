"""Images as training rows: decoding, geometry, augmentation and caption handling, each a plain function of a row and a key.

``decode``          bytes / path / PIL image / array -> float32 ``[H, W, 3]`` in [-1, 1]
``resize_shorter``  the shorter side to ``size`` (area filter down, bicubic up), keeping the aspect
``center_crop`` / ``random_crop`` / ``random_flip``   geometry; the random ones draw from the row's key, so a row augments the
                    same way whichever worker, rank or epoch position reads it
``bucketed``        aspect-ratio buckets: the bucket of area ``size^2`` whose aspect is nearest the image's (multiples of 64)
``caption_dropout`` the caption replaced by the empty string with probability ``p`` (classifier-free guidance training)
``ImageFolder``     a directory of images with sidecar captions (``x.jpg`` + ``x.txt`` or a ``captions.jsonl``)
``Augment``         a chainable map stage composed of the above

Reference: src/dew/data/images.py, src/dew/data/image_augmentation.py (decode / resize / crop / flip, caption dropout, aspect
buckets).
"""
from __future__ import annotations

import hashlib
import io
import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import numpy as np

from .dataset import Dataset

EXTENSIONS = (".jpg", ".jpeg", ".png", ".webp", ".bmp")


def row_key(row: Mapping[str, Any], salt: int = 0) -> int:
    """A stable 63-bit key of a row: its ``key`` / ``id`` / ``path`` field, else a hash of its caption and image shape."""
    for name in ("key", "id", "path", "__key__"):
        if name in row:
            basis = str(row[name])
            break
    else:
        img = row.get("image")
        basis = f"{row.get('caption', '')}|{getattr(img, 'shape', None)}"
    h = hashlib.blake2b(f"{salt}:{basis}".encode(), digest_size=8).digest()
    return int.from_bytes(h, "little") & 0x7FFFFFFFFFFFFFFF


def decode(image: Any) -> np.ndarray:
    from PIL import Image
    if isinstance(image, np.ndarray):
        arr = image
        if arr.dtype == np.uint8:
            arr = arr.astype(np.float32) / 127.5 - 1.0
        arr = arr.astype(np.float32)
        if arr.ndim == 2:
            arr = np.repeat(arr[..., None], 3, -1)
        return arr[..., :3]
    if isinstance(image, (bytes, bytearray)):
        image = Image.open(io.BytesIO(bytes(image)))
    elif isinstance(image, (str, os.PathLike)):
        image = Image.open(image)
    if not isinstance(image, Image.Image):
        raise TypeError(f"cannot decode an image from {type(image).__name__}")
    return np.asarray(image.convert("RGB"), dtype=np.float32) / 127.5 - 1.0


def _resize(arr: np.ndarray, height: int, width: int) -> np.ndarray:
    from PIL import Image
    if arr.shape[:2] == (height, width):
        return arr
    down = height * width < arr.shape[0] * arr.shape[1]
    chans = [Image.fromarray(arr[..., c]).resize((width, height), Image.BOX if down else Image.BICUBIC) for c in range(arr.shape[-1])]
    return np.stack([np.asarray(c, dtype=np.float32) for c in chans], -1).clip(-1.0, 1.0)


def resize_shorter(arr: np.ndarray, size: int) -> np.ndarray:
    h, w = arr.shape[:2]
    scale = size / min(h, w)
    return _resize(arr, max(size, round(h * scale)), max(size, round(w * scale)))


def center_crop(arr: np.ndarray, height: int, width: Optional[int] = None) -> np.ndarray:
    width = width or height
    h, w = arr.shape[:2]
    top, left = max(0, (h - height) // 2), max(0, (w - width) // 2)
    return arr[top:top + height, left:left + width]


def random_crop(arr: np.ndarray, height: int, width: Optional[int], key: int) -> Tuple[np.ndarray, Tuple[int, int]]:
    width = width or height
    h, w = arr.shape[:2]
    rng = np.random.default_rng(key)
    top = int(rng.integers(0, max(1, h - height + 1)))
    left = int(rng.integers(0, max(1, w - width + 1)))
    return arr[top:top + height, left:left + width], (top, left)


def random_flip(arr: np.ndarray, key: int, p: float = 0.5) -> Tuple[np.ndarray, bool]:
    flip = bool(np.random.default_rng(key ^ 0x5F3759DF).random() < p)
    return (arr[:, ::-1].copy() if flip else arr), flip


def buckets(size: int, step: int = 64, max_aspect: float = 2.0) -> List[Tuple[int, int]]:
    """(height, width) buckets of area about ``size^2``, sides multiples of ``step``, aspects within ``max_aspect``."""
    out = set()
    w = step
    while w <= size * max_aspect:
        h = max(step, int(round(size * size / w / step)) * step)
        if max(h / w, w / h) <= max_aspect + 1e-6:
            out.add((h, w))
        w += step
    return sorted(out)


def bucketed(arr: np.ndarray, table: Sequence[Tuple[int, int]]) -> Tuple[np.ndarray, Tuple[int, int]]:
    """``arr`` resized to cover, then centre-cropped to, the bucket whose aspect is nearest its own (in log space)."""
    h, w = arr.shape[:2]
    aspect = np.log(h / w)
    bh, bw = min(table, key=lambda b: abs(np.log(b[0] / b[1]) - aspect))
    scale = max(bh / h, bw / w)
    arr = _resize(arr, max(bh, round(h * scale)), max(bw, round(w * scale)))
    return center_crop(arr, bh, bw), (bh, bw)


def caption_dropout(caption: str, key: int, p: float = 0.1) -> str:
    return "" if np.random.default_rng(key ^ 0x9E3779B9).random() < p else caption


@dataclass
class Augment:
    size: int = 256
    crop: str = "center"           # center | random | bucket
    flip: bool = False
    drop_caption: float = 0.0
    image_key: str = "image"
    out_key: str = "sample"
    salt: int = 0

    def __post_init__(self):
        if self.crop not in ("center", "random", "bucket"):
            raise ValueError(f"crop is center, random or bucket, got {self.crop!r}")
        self._table = buckets(self.size) if self.crop == "bucket" else None

    def __call__(self, row: Mapping[str, Any]) -> Dict[str, Any]:
        key = row_key(row, self.salt)
        arr = decode(row[self.image_key])
        out = {k: v for k, v in row.items() if k != self.image_key}
        original = arr.shape[:2]
        if self.crop == "bucket":
            arr, bucket = bucketed(arr, self._table)
            out["bucket"] = bucket
            origin = (0, 0)
        else:
            arr = resize_shorter(arr, self.size)
            if self.crop == "random":
                arr, origin = random_crop(arr, self.size, self.size, key)
            else:
                h, w = arr.shape[:2]
                origin = (max(0, (h - self.size) // 2), max(0, (w - self.size) // 2))
                arr = center_crop(arr, self.size)
        if self.flip:
            arr, flipped = random_flip(arr, key)
            out["flipped"] = flipped
        if "caption" in out and self.drop_caption > 0:
            out["caption"] = caption_dropout(out["caption"], key, self.drop_caption)
        out[self.out_key] = np.ascontiguousarray(arr)
        out["original_size"], out["crop_origin"] = np.array(original), np.array(origin)     # SDXL-style size conditioning
        return out


class ImageFolder(Dataset):
    """Images under ``root`` (recursively), each with its caption from ``<stem>.txt`` beside it or from ``captions.jsonl`` rows
    ``{"file": ..., "caption": ...}``; rows are ``{"path", "image" (the path, decoded lazily by ``Augment``), "caption"}``."""

    def __init__(self, root: str, captions: Optional[str] = None):
        paths = sorted(os.path.join(d, f) for d, _, fs in os.walk(root) for f in fs if f.lower().endswith(EXTENSIONS))
        table: Dict[str, str] = {}
        captions = captions or os.path.join(root, "captions.jsonl")
        if os.path.exists(captions):
            with open(captions) as f:
                for line in f:
                    if line.strip():
                        rec = json.loads(line)
                        table[os.path.normpath(os.path.join(root, rec["file"]))] = rec.get("caption", "")
        self.root, self._paths, self._table = root, paths, table
        super().__init__(records=None, length=len(paths))

    def _get(self, i: int):
        path = self._paths[i]
        caption = self._table.get(os.path.normpath(path))
        if caption is None:
            side = os.path.splitext(path)[0] + ".txt"
            caption = open(side).read().strip() if os.path.exists(side) else ""
        return {"path": os.path.relpath(path, self.root), "image": path, "caption": caption}
