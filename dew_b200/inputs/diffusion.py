"""Image preprocessing and image conditions for latent diffusion: the CLIP image transform as tensor arithmetic, and an
inpainting run's mask and masked latents.

``CLIPImageTransform``      uint8 NHWC pixels -> the tower's input: bicubic resize of the shorter side to ``size`` (antialiased),
                            centre crop, scale to [0, 1], normalise by the published mean / std; NCHW float32
``latent_image_conditions`` pixels in [-1, 1] and a binary pixel mask (1 = repaint) -> ``mask [B, h, w, 1]`` on the latent grid
                            (nearest) and ``masked_image [B, h, w, C]`` = the autoencoder's encoding of the pixels with the masked
                            region blanked; both stay present in the conditional and the unconditional guidance branch
``blend_known``             during sampling, the known region of the latents is reset to the (noised) original after every step

Reference: src/dew/inputs/diffusion.py (``CLIPImageTransform``, ``latent_image_conditions``).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


class CLIPImageTransform:
    def __init__(self, size: int = 224, mean: Sequence[float] = CLIP_MEAN, std: Sequence[float] = CLIP_STD):
        self.size, self.mean, self.std = size, tuple(mean), tuple(std)

    def __call__(self, pixels: torch.Tensor) -> torch.Tensor:
        """``pixels [B, H, W, 3]`` with integer levels 0..255 in any dtype -> ``[B, 3, size, size]`` float32."""
        x = pixels.permute(0, 3, 1, 2).to(torch.float32)
        B, C, H, W = x.shape
        scale = self.size / min(H, W)
        nh, nw = max(self.size, round(H * scale)), max(self.size, round(W * scale))
        if (nh, nw) != (H, W):
            x = F.interpolate(x, size=(nh, nw), mode="bicubic", antialias=True, align_corners=False).clamp(0, 255).round()
        top, left = (nh - self.size) // 2, (nw - self.size) // 2
        x = x[:, :, top:top + self.size, left:left + self.size] / 255.0
        mean = torch.tensor(self.mean, device=x.device).view(1, 3, 1, 1)
        std = torch.tensor(self.std, device=x.device).view(1, 3, 1, 1)
        return (x - mean) / std


def latent_image_conditions(pixels: torch.Tensor, mask: torch.Tensor, autoencoder, generator=None) -> Dict[str, torch.Tensor]:
    """``pixels [B, H, W, C]`` in [-1, 1], ``mask [B, H, W]`` or ``[B, H, W, 1]`` (1 = repaint)."""
    m = mask.float()
    if m.dim() == 3:
        m = m[..., None]
    m = (m > 0.5).float()
    with torch.no_grad():
        masked = autoencoder.encode(pixels * (1 - m))
    h, w = masked.shape[1], masked.shape[2]
    small = F.interpolate(m.permute(0, 3, 1, 2), size=(h, w), mode="nearest").permute(0, 2, 3, 1)
    return {"mask": small, "masked_image": masked}


def blend_known(latents: torch.Tensor, original: torch.Tensor, mask: torch.Tensor, noise: torch.Tensor, alpha: float, sigma: float) -> torch.Tensor:
    """Keep the repainted region of ``latents`` and reset the known region to the original latents at the current noise level
    (``alpha x0 + sigma noise``): what an inpainting sampler does after every step when the model takes no mask input."""
    known = alpha * original + sigma * noise
    return mask * latents + (1 - mask) * known
