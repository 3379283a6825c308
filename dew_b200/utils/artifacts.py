"""Artifacts a run can log: image / video grids, text samples, representations, token scores
(reference: src/dew/artifacts.py)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Optional, Sequence

import torch


def uint8_pixels(x: torch.Tensor) -> torch.Tensor:
    """[-1, 1] floats -> uint8."""
    return ((x.float().clamp(-1, 1) + 1) * 127.5).round().to(torch.uint8)


@dataclass
class ImageGrid:
    images: torch.Tensor            # [N, H, W, C] in [-1, 1]
    columns: Optional[int] = None
    captions: Optional[Sequence[str]] = None

    def grid(self) -> torch.Tensor:
        n, h, w, c = self.images.shape
        cols = self.columns or max(1, int(n ** 0.5))
        rows = (n + cols - 1) // cols
        canvas = torch.zeros(rows * h, cols * w, c, dtype=torch.uint8)
        px = uint8_pixels(self.images).cpu()
        for i in range(n):
            r, cc = divmod(i, cols)
            canvas[r * h:(r + 1) * h, cc * w:(cc + 1) * w] = px[i]
        return canvas

    def save(self, path) -> None:
        """Binary PPM/PGM: needs no imaging library."""
        g = self.grid()
        h, w, c = g.shape
        header = (f"P6\n{w} {h}\n255\n" if c == 3 else f"P5\n{w} {h}\n255\n").encode()
        data = g[..., :3].contiguous().numpy().tobytes() if c >= 3 else g[..., 0].contiguous().numpy().tobytes()
        with open(path, "wb") as f:
            f.write(header + data)


@dataclass
class VideoGrid:
    videos: torch.Tensor            # [N, T, H, W, C]
    fps: int = 8

    def frames(self) -> List[ImageGrid]:
        return [ImageGrid(self.videos[:, t]) for t in range(self.videos.shape[1])]


@dataclass
class TextSamples:
    prompts: Sequence[str]
    completions: Sequence[str]

    def rows(self):
        return [{"prompt": p, "completion": c} for p, c in zip(self.prompts, self.completions)]


@dataclass
class Representations:
    features: torch.Tensor
    labels: Optional[torch.Tensor] = None


@dataclass
class TokenScores:
    tokens: Sequence[Sequence[str]]
    scores: Sequence[Sequence[float]]
