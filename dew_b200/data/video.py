"""Video clips as training rows: frame arrays in, fixed-length clips out.

``clip_starts(frames, length, stride, count, key)``   where clips of ``length`` frames taken every ``stride`` frames may start, and
                                                      ``count`` of them drawn by the row's key (all of them in order with ``count=None``)
``clips(video, ...)``                                 the clips ``[count, length, H, W, C]``, with their first-frame indices and the
                                                      frame rate the stride leaves
``Clips``                                             a chainable map stage; the last clip of a short video is padded by repeating
                                                      its last frame, with a ``frames_mask``

Reference: src/dew/data/video.py (clip sampling with stride and padding masks).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

import numpy as np

from .images import row_key


def clip_starts(frames: int, length: int, stride: int = 1, count: Optional[int] = None, key: int = 0) -> np.ndarray:
    span = (length - 1) * stride + 1
    last = frames - span
    if last < 0:
        return np.zeros(1, dtype=np.int64)
    starts = np.arange(0, last + 1)
    if count is None:
        return starts[:: max(1, span)]
    rng = np.random.default_rng(key)
    return np.sort(rng.choice(starts, size=min(count, len(starts)), replace=False)) if len(starts) >= count else np.sort(rng.choice(starts, size=count))


def clips(video: np.ndarray, length: int, stride: int = 1, count: Optional[int] = None, key: int = 0, fps: Optional[float] = None
          ) -> Dict[str, np.ndarray]:
    T = video.shape[0]
    starts = clip_starts(T, length, stride, count, key)
    idx = starts[:, None] + np.arange(length)[None] * stride
    mask = idx < T
    out = {"clip": video[np.minimum(idx, T - 1)], "first_frame": starts, "frames_mask": mask}
    if fps is not None:
        out["fps"] = np.full(len(starts), fps / stride, dtype=np.float32)
    return out


@dataclass
class Clips:
    length: int = 16
    stride: int = 1
    count: Optional[int] = 1
    video_key: str = "video"
    salt: int = 0

    def __call__(self, row: Mapping[str, Any]) -> Dict[str, Any]:
        out = {k: v for k, v in row.items() if k != self.video_key}
        got = clips(np.asarray(row[self.video_key]), self.length, self.stride, self.count, row_key(row, self.salt), row.get("fps"))
        if self.count == 1:
            got = {k: v[0] for k, v in got.items()}
        out.update(got)
        return out
