"""The gate-race front camera: an analytic scene (checker ground, yawed boxes, upright cylinders, gradient sky) ray cast
into a headless image buffer ``[B, H, W, 3]`` - by the CUDA kernel ``dewb_raycast`` on a GPU, by ``render_reference``
(the same math in fp32 torch: oracle and timed CPU baseline) anywhere.

The lens is a pinhole or an equidistant fisheye cast directly; ``fisheye_map`` / ``fisheyed`` give the other route the
reference takes (draw a pinhole, resample it).  Motion blur averages one ray per shutter pose (two poses by default).

Reference: src/dew/rl/hyperlux.py:43-78 (``fisheye_map``, ``fisheyed``), :90-260 (``HyperLuxRenderer`` over an external
OptiX ray tracer; graphics-API renderers are unavailable on this class of machine, so the scene is analytic here).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

SUN = (0.3713907, 0.2785430, 0.8863914)


@dataclass
class Camera:
    size: Tuple[int, int] = (96, 96)        # (H, W)
    fov: float = 120.0                      # horizontal field of view, degrees
    fisheye: bool = True
    fog: float = 0.02
    checker: float = 1.0
    samples: int = 2                        # shutter poses averaged (motion blur)


def look_at(position: torch.Tensor, target: torch.Tensor, up=(0.0, 0.0, 1.0)) -> torch.Tensor:
    """Camera rows ``[..., 12]``: position, then right / down / forward axes in the world frame."""
    f = torch.nn.functional.normalize(target - position, dim=-1)
    upv = torch.tensor(up, dtype=position.dtype, device=position.device).expand_as(f)
    r = torch.nn.functional.normalize(torch.cross(f, upv, dim=-1), dim=-1)
    d = torch.cross(f, r, dim=-1)
    return torch.cat([position, r, d, f], -1)


def gate_boxes(center: torch.Tensor, yaw: torch.Tensor, inner: float = 1.0, bar: float = 0.15, depth: float = 0.1,
               color=(0.9, 0.3, 0.1)) -> torch.Tensor:
    """A square gate (opening ``inner`` wide, frame bars ``bar`` thick) facing along its yaw, as 4 boxes ``[..., 4, 10]``:
    the frame lies in the plane spanned by the gate's local y axis and world z."""
    h = inner / 2 + bar / 2
    c, s = torch.cos(yaw), torch.sin(yaw)
    zeros = torch.zeros_like(yaw)
    out = []
    for (dy, dz, hy, hz) in ((0.0, h, inner / 2 + bar, bar / 2), (0.0, -h, inner / 2 + bar, bar / 2),
                             (h, 0.0, bar / 2, inner / 2), (-h, 0.0, bar / 2, inner / 2)):
        cx = center[..., 0] - s * dy
        cy = center[..., 1] + c * dy
        cz = center[..., 2] + dz
        row = [cx, cy, cz, zeros + depth / 2, zeros + hy, zeros + hz, yaw] + [zeros + v for v in color]
        out.append(torch.stack(row, -1))
    return torch.stack(out, -2)


def _rays(cam: Camera, device, dtype=torch.float32):
    H, W = cam.size
    u = ((torch.arange(W, device=device, dtype=dtype) + 0.5) / W * 2 - 1)[None, :].expand(H, W)
    v = ((torch.arange(H, device=device, dtype=dtype) + 0.5) / H * 2 - 1)[:, None].expand(H, W)
    half = math.radians(cam.fov) / 2
    if cam.fisheye:
        rad = torch.sqrt(u * u + v * v)
        theta = half * rad
        held = theta < 1.5607963
        k = torch.where(rad > 1e-12, torch.sin(theta) / rad.clamp_min(1e-12), torch.zeros_like(rad))
        d = torch.stack([u * k, v * k, torch.cos(theta)], -1)
    else:
        d = torch.stack([u * math.tan(half), v * math.tan(half) * (H / W), torch.ones_like(u)], -1)
        d = d / d.norm(dim=-1, keepdim=True)
        held = torch.ones_like(u, dtype=torch.bool)
    return d, held


def render_reference(cameras: torch.Tensor, boxes: torch.Tensor, cylinders: torch.Tensor, cam: Camera) -> torch.Tensor:
    """fp32 torch restatement of the kernel.  cameras ``[B, samples, 12]``, boxes ``[B, nb, 10]``, cylinders ``[B, nc, 7]``."""
    B = cameras.shape[0]
    dev = cameras.device
    H, W = cam.size
    dcam, held = _rays(cam, dev)
    inf = torch.tensor(1e30, device=dev)
    sun = torch.tensor(SUN, device=dev)
    acc = torch.zeros(B, H, W, 3, device=dev)
    for s in range(cameras.shape[1]):
        c = cameras[:, s].float()
        o = c[:, None, None, 0:3]
        R = c[:, 3:12].reshape(B, 3, 3)                                   # rows: right, down, forward
        d = torch.einsum("hwk,bkx->bhwx", dcam, R)
        ox, oy, oz = o[..., 0], o[..., 1], o[..., 2]
        dx, dy, dz = d[..., 0], d[..., 1], d[..., 2]
        t = inf.expand(B, H, W).clone()
        normal = torch.zeros(B, H, W, 3, device=dev); normal[..., 2] = 1
        color = torch.zeros(B, H, W, 3, device=dev)
        ground = (dz < -1e-6) & (oz > 0)
        tg = torch.where(ground, -oz / torch.where(ground, dz, -torch.ones_like(dz)), inf)
        gx, gy = ox + tg * dx, oy + tg * dy
        cell = ((torch.floor(gx / cam.checker).to(torch.int64) + torch.floor(gy / cam.checker).to(torch.int64)) & 1).bool()
        shade = torch.where(cell, torch.full_like(tg, 0.55), torch.full_like(tg, 0.35))
        t = torch.where(ground, tg, t)
        color = torch.where(ground[..., None], torch.stack([shade * 0.9, shade, shade * 0.8], -1), color)
        any_hit = ground.clone()
        for i in range(boxes.shape[1]):
            bx = boxes[:, i].float()[:, None, None, :]
            cy, sy = torch.cos(bx[..., 6]), torch.sin(bx[..., 6])
            px, py, pz = ox - bx[..., 0], oy - bx[..., 1], oz - bx[..., 2]
            lo = torch.stack([cy * px + sy * py, -sy * px + cy * py, pz.expand_as(px)], -1)
            dl = torch.stack([cy * dx + sy * dy, -sy * dx + cy * dy, dz], -1)
            hf = bx[..., 3:6].expand_as(lo)
            par = dl.abs() < 1e-12
            inv = 1.0 / torch.where(par, torch.ones_like(dl), dl)
            ta, tb = (-hf - lo) * inv, (hf - lo) * inv
            sg = torch.where(ta > tb, torch.ones_like(ta), -torch.ones_like(ta))
            tmin, tmax = torch.minimum(ta, tb), torch.maximum(ta, tb)
            outside = par & (lo.abs() > hf)
            tmin = torch.where(par, torch.full_like(tmin, -1e30), tmin)
            tmax = torch.where(par, torch.full_like(tmax, 1e30), tmax)
            t0, axis = tmin.max(-1)
            t1 = torch.minimum(tmax.min(-1).values, t)
            hit = (~outside.any(-1)) & (t0 <= t1) & (t0 > 1e-4) & (t0 < t) & (t0 > 0)
            sign = sg.gather(-1, axis[..., None]).squeeze(-1)
            nl = torch.nn.functional.one_hot(axis, 3).float() * sign[..., None]
            nw = torch.stack([cy * nl[..., 0] - sy * nl[..., 1], sy * nl[..., 0] + cy * nl[..., 1], nl[..., 2]], -1)
            t = torch.where(hit, t0, t)
            normal = torch.where(hit[..., None], nw, normal)
            color = torch.where(hit[..., None], bx[..., 7:10].expand_as(color), color)
            any_hit |= hit
        for i in range(cylinders.shape[1]):
            cyl = cylinders[:, i].float()[:, None, None, :]
            px, py = ox - cyl[..., 0], oy - cyl[..., 1]
            a = dx * dx + dy * dy
            b = px * dx + py * dy
            cc = px * px + py * py - cyl[..., 2] ** 2
            disc = b * b - a * cc
            ok = (a >= 1e-12) & (disc >= 0)
            tc = (-b - torch.sqrt(disc.clamp_min(0))) / torch.where(a >= 1e-12, a, torch.ones_like(a))
            z = oz + tc * dz
            hit = ok & (tc > 1e-4) & (tc < t) & (z >= 0) & (z <= cyl[..., 3])
            nw = torch.stack([(px + tc * dx) / cyl[..., 2], (py + tc * dy) / cyl[..., 2], torch.zeros_like(tc)], -1)
            t = torch.where(hit, tc, t)
            normal = torch.where(hit[..., None], nw, normal)
            color = torch.where(hit[..., None], cyl[..., 4:7].expand_as(color), color)
            any_hit |= hit
        up = dz.clamp(0, 1)
        sky = torch.stack([0.65 - 0.35 * up, 0.78 - 0.28 * up, 0.95 - 0.10 * up], -1)
        light = 0.35 + 0.65 * (normal * sun).sum(-1).clamp_min(0)
        f = torch.exp(-cam.fog * torch.where(any_hit, t, torch.zeros_like(t)))[..., None]
        lit = f * color * light[..., None] + (1 - f) * sky
        acc += torch.where(any_hit[..., None], lit, sky)
    img = acc / cameras.shape[1]
    return torch.where(held[None, ..., None], img, torch.zeros_like(img))


def render(cameras: torch.Tensor, boxes: torch.Tensor, cylinders: torch.Tensor, cam: Camera, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Images ``[B, H, W, 3]`` fp32 in [0, 1]: the CUDA ray caster for CUDA tensors, the torch restatement otherwise."""
    if not cameras.is_cuda:
        return render_reference(cameras, boxes, cylinders, cam)
    from ..ops import library as L
    B, H, W = cameras.shape[0], cam.size[0], cam.size[1]
    cameras, boxes, cylinders = cameras.float().contiguous(), boxes.float().contiguous(), cylinders.float().contiguous()
    if out is None:
        out = torch.empty(B, H, W, 3, device=cameras.device, dtype=torch.float32)
    rc = L.load().dewb_raycast(L.ptr(cameras), L.ptr(boxes), L.ptr(cylinders), L.ptr(out), ctypes.c_int(B), ctypes.c_int(H), ctypes.c_int(W),
                               ctypes.c_int(cameras.shape[1]), ctypes.c_int(boxes.shape[1]), ctypes.c_int(cylinders.shape[1]),
                               ctypes.c_float(cam.fov), ctypes.c_int(int(cam.fisheye)), ctypes.c_float(cam.fog), ctypes.c_float(cam.checker),
                               L.stream_ptr())
    L.check(rc, "raycast")
    L.count_launches()
    return out


def fisheye_map(size: int, source: int, fov: float):
    """Where each pixel of a ``size``-square equidistant fisheye of horizontal field of view ``fov`` samples a
    ``source``-square pinhole image of the same field of view: four corner indices ``[size, size, 4]`` (row * source +
    column), their bilinear weights (0 where the pinhole does not hold the direction) and the held mask."""
    half = math.radians(fov) / 2
    centers = (torch.arange(size, dtype=torch.float64) + 0.5) / size * 2 - 1
    down, right = torch.meshgrid(centers, centers, indexing="ij")
    radius = torch.hypot(right, down)
    theta = half * radius
    tangent = torch.tan(theta.clamp_max(math.pi / 2 - 1e-6)) / radius.clamp_min(1e-12) / math.tan(half)
    across, along = right * tangent, down * tangent
    held = (theta < math.pi / 2) & (across.abs() <= 1) & (along.abs() <= 1)
    column, row = (across + 1) / 2 * source - 0.5, (along + 1) / 2 * source - 0.5
    left, top = torch.floor(column), torch.floor(row)
    dx, dy = column - left, row - top
    corners, weights = [], []
    for oy, wy in ((0, 1 - dy), (1, dy)):
        for ox, wx in ((0, 1 - dx), (1, dx)):
            r = (top + oy).clamp(0, source - 1).long()
            c = (left + ox).clamp(0, source - 1).long()
            corners.append(r * source + c)
            weights.append(torch.where(held, wy * wx, torch.zeros_like(wx)))
    return torch.stack(corners, -1), torch.stack(weights, -1).float(), held


def fisheyed(images: torch.Tensor, corners: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """Pinhole images ``[B, S, S, C]`` resampled to a fisheye ``[B, N, N, C]`` by ``fisheye_map``'s corners and weights."""
    B, C = images.shape[0], images.shape[-1]
    flat = images.reshape(B, -1, C).float()
    n = corners.shape[0]
    picked = flat[:, corners.reshape(-1).to(images.device)].reshape(B, n * n, 4, C)
    return (picked * weights.reshape(1, n * n, 4, 1).to(images.device)).sum(2).reshape(B, n, n, C)
