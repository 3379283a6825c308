"""Evaluation metrics: PSNR, SSIM, Frechet distance between feature sets (FID given an encoder), CLIP-style cosine
score, perplexity and expected calibration error (reference: src/dew/eval - FID, CLIPScore, PSNR, SSIM, LPIPS,
lm-eval harness, calibration)."""
from __future__ import annotations

import math
from typing import Callable, Optional, Sequence

import torch
import torch.nn.functional as F


def psnr(a: torch.Tensor, b: torch.Tensor, data_range: float = 2.0) -> torch.Tensor:
    mse = ((a.float() - b.float()) ** 2).reshape(a.shape[0], -1).mean(1)
    return 10 * torch.log10(data_range ** 2 / mse.clamp_min(1e-12))


def ssim(a: torch.Tensor, b: torch.Tensor, data_range: float = 2.0, window: int = 7) -> torch.Tensor:
    """Mean structural similarity of NHWC images with a uniform window."""
    x, y = a.float().permute(0, 3, 1, 2), b.float().permute(0, 3, 1, 2)
    C = x.shape[1]
    k = torch.ones(C, 1, window, window, device=x.device) / window ** 2
    mu_x, mu_y = F.conv2d(x, k, groups=C), F.conv2d(y, k, groups=C)
    sx = F.conv2d(x * x, k, groups=C) - mu_x ** 2
    sy = F.conv2d(y * y, k, groups=C) - mu_y ** 2
    sxy = F.conv2d(x * y, k, groups=C) - mu_x * mu_y
    c1, c2 = (0.01 * data_range) ** 2, (0.03 * data_range) ** 2
    s = ((2 * mu_x * mu_y + c1) * (2 * sxy + c2)) / ((mu_x ** 2 + mu_y ** 2 + c1) * (sx + sy + c2))
    return s.reshape(s.shape[0], -1).mean(1)


def _sqrtm_psd(m: torch.Tensor) -> torch.Tensor:
    w, v = torch.linalg.eigh(m.double())
    return (v * w.clamp_min(0).sqrt()) @ v.T


def frechet_distance(feat_a: torch.Tensor, feat_b: torch.Tensor) -> float:
    """||mu_a - mu_b||^2 + Tr(Ca + Cb - 2 (Ca^1/2 Cb Ca^1/2)^1/2) over feature rows."""
    a, b = feat_a.double(), feat_b.double()
    mu_a, mu_b = a.mean(0), b.mean(0)
    ca, cb = torch.cov(a.T), torch.cov(b.T)
    ra = _sqrtm_psd(ca)
    cross = _sqrtm_psd(ra @ cb @ ra)
    return float(((mu_a - mu_b) ** 2).sum() + torch.trace(ca) + torch.trace(cb) - 2 * torch.trace(cross))


def fid(images_a: torch.Tensor, images_b: torch.Tensor, encoder: Callable[[torch.Tensor], torch.Tensor]) -> float:
    with torch.no_grad():
        return frechet_distance(encoder(images_a), encoder(images_b))


def lpips(a: torch.Tensor, b: torch.Tensor, features: Callable[[torch.Tensor], Sequence[torch.Tensor]],
          weights: Optional[Sequence[torch.Tensor]] = None) -> torch.Tensor:
    """Learned perceptual image patch similarity (Zhang et al. 2018) per pair: ``features(images NHWC in [-1, 1])`` returns the
    chosen layers' activations ``[B, C_l, H_l, W_l]`` (a frozen AlexNet / VGG loaded by the caller: no weights ship here);
    each is unit-normalised over channels, the squared difference weighted per channel (``weights[l] [C_l]``, uniform when
    None), averaged over space and summed over layers."""
    fa, fb = features(a), features(b)
    total = torch.zeros(a.shape[0], device=a.device)
    for i, (x, y) in enumerate(zip(fa, fb)):
        x = x.float() / x.float().pow(2).sum(1, keepdim=True).add(1e-10).sqrt()
        y = y.float() / y.float().pow(2).sum(1, keepdim=True).add(1e-10).sqrt()
        d = (x - y) ** 2
        w = torch.full((x.shape[1],), 1.0 / x.shape[1], device=x.device) if weights is None else weights[i].to(x.device).float()
        total = total + (d * w[None, :, None, None]).sum(1).mean((1, 2))
    return total


def clip_score(image_features: torch.Tensor, text_features: torch.Tensor) -> torch.Tensor:
    return 100 * F.cosine_similarity(image_features.float(), text_features.float(), dim=-1).clamp_min(0)


def perplexity(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> float:
    nll = F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), targets.reshape(-1), ignore_index=ignore_index)
    return float(torch.exp(nll))


def expected_calibration_error(probs: torch.Tensor, labels: torch.Tensor, bins: int = 15) -> float:
    conf, pred = probs.max(-1)
    acc = (pred == labels).float()
    edges = torch.linspace(0, 1, bins + 1, device=probs.device)
    ece = torch.zeros((), device=probs.device)
    for lo, hi in zip(edges[:-1], edges[1:]):
        m = (conf > lo) & (conf <= hi)
        if bool(m.any()):
            ece = ece + m.float().mean() * (acc[m].mean() - conf[m].mean()).abs()
    return float(ece)
