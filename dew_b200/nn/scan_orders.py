"""Patch grids as token sequences: the 2-D sin-cos position signal and the orders a grid can be read in - raster, zigzag (every other
row reversed, so consecutive tokens are always neighbours) and a generalised Hilbert curve for any rectangle (consecutive tokens are
neighbours and nearby tokens stay nearby in the sequence, which is what a recurrent or windowed mixer over patches wants).  An order is a
permutation of the row-major patch index; it depends on the grid alone, so it is built once on the host and cached.

Reference: src/dew/nn/scan_orders.py.
"""
from __future__ import annotations

import functools
from typing import List, Tuple

import torch


def sincos_2d(height: int, width: int, dim: int, max_period: float = 10000.0) -> torch.Tensor:
    """``[height * width, dim]`` row-major: half of the channels encode the row, half the column, each as sin | cos over
    ``dim / 4`` geometric frequencies."""
    if dim % 4:
        raise ValueError(f"the 2-D sin-cos signal splits its channels in four; {dim} does not divide")
    freq = max_period ** (-torch.arange(dim // 4, dtype=torch.float64) / (dim // 4))
    ys, xs = torch.meshgrid(torch.arange(height, dtype=torch.float64), torch.arange(width, dtype=torch.float64), indexing="ij")

    def axis(p):
        ang = p.reshape(-1, 1) * freq
        return torch.cat([ang.sin(), ang.cos()], 1)
    return torch.cat([axis(ys), axis(xs)], 1).float()


def raster(height: int, width: int) -> torch.Tensor:
    return torch.arange(height * width)


def zigzag(height: int, width: int) -> torch.Tensor:
    rows = torch.arange(height * width).view(height, width).clone()
    rows[1::2] = rows[1::2].flip(1)
    return rows.reshape(-1)


def _sign(v: int) -> int:
    return (v > 0) - (v < 0)


def _curve(x: int, y: int, ax: int, ay: int, bx: int, by: int, out: List[Tuple[int, int]]) -> None:
    """Fill the rectangle spanned from (x, y) by the major axis (ax, ay) and the minor axis (bx, by) with a path of unit steps."""
    w, h = abs(ax + ay), abs(bx + by)
    dax, day, dbx, dby = _sign(ax), _sign(ay), _sign(bx), _sign(by)
    if h == 1:
        for _ in range(w):
            out.append((x, y))
            x, y = x + dax, y + day
        return
    if w == 1:
        for _ in range(h):
            out.append((x, y))
            x, y = x + dbx, y + dby
        return
    ax2, ay2, bx2, by2 = ax // 2, ay // 2, bx // 2, by // 2
    w2, h2 = abs(ax2 + ay2), abs(bx2 + by2)
    if 2 * w > 3 * h:                                           # long rectangle: split the major axis only
        if w2 % 2 and w > 2:
            ax2, ay2 = ax2 + dax, ay2 + day
        _curve(x, y, ax2, ay2, bx, by, out)
        _curve(x + ax2, y + ay2, ax - ax2, ay - ay2, bx, by, out)
        return
    if h2 % 2 and h > 2:
        bx2, by2 = bx2 + dbx, by2 + dby
    _curve(x, y, bx2, by2, ax2, ay2, out)
    _curve(x + bx2, y + by2, ax, ay, bx - bx2, by - by2, out)
    _curve(x + (ax - dax) + (bx2 - dbx), y + (ay - day) + (by2 - dby), -bx2, -by2, -(ax - ax2), -(ay - ay2), out)


@functools.lru_cache(maxsize=64)
def _hilbert(height: int, width: int) -> Tuple[int, ...]:
    path: List[Tuple[int, int]] = []
    if width >= height:
        _curve(0, 0, width, 0, 0, height, path)
    else:
        _curve(0, 0, 0, height, width, 0, path)
    return tuple(y * width + x for x, y in path)


def hilbert(height: int, width: int) -> torch.Tensor:
    """A space-filling order of any ``height x width`` grid: every step moves to a 4-neighbour (8-neighbour at a few joints of odd-sized
    rectangles), and the curve recursively fills compact sub-rectangles."""
    return torch.tensor(_hilbert(height, width), dtype=torch.long)


ORDERS = {"raster": raster, "zigzag": zigzag, "hilbert": hilbert}


def order(name: str, height: int, width: int) -> torch.Tensor:
    if name not in ORDERS:
        raise KeyError(f"scan order {name!r}; known: {sorted(ORDERS)}")
    return ORDERS[name](height, width)


def inverse(perm: torch.Tensor) -> torch.Tensor:
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), device=perm.device)
    return inv


def reorder(tokens: torch.Tensor, perm: torch.Tensor) -> torch.Tensor:
    """``tokens [B, N, ...]`` in row-major order -> in the order ``perm`` reads the grid; ``reorder(y, inverse(perm))`` puts them back."""
    return tokens.index_select(1, perm.to(tokens.device))
