"""Image and audio conditioning around the shared causal decoder.

``VisionLanguageModel``   a vision tower, a projector and a decoder: every image's patch features are projected to the decoder's width
                          and written over the positions its placeholder tokens hold (LLaVA's scheme: ``<image>`` repeated once per
                          patch), then the decoder runs as on text.  The loss, generation and serving paths are the decoder's own.
``Projector``             linear, two-layer MLP (GELU) or a pixel-shuffle merger that folds ``s x s`` neighbouring patches into one token
``AudioEncoder``          log-mel frames -> two strided convolutions (4 x fewer frames) -> transformer blocks: a Whisper-shaped encoder
                          whose outputs splice into the decoder the same way (placeholder ``<audio>`` tokens)
``log_mel``               waveform -> log-mel spectrogram (Hann window STFT, a triangular mel filter bank, log10 with the dynamic
                          range clamp speech models use)
``expand_placeholders``   a prompt's single ``<image>`` token repeated to one per patch

Reference: src/dew/nn/multimodal.py (image and audio conditioning around the decoder), src/dew/nn/audio.py.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .encoders import EncoderConfig, TransformerEncoder


class Projector(nn.Module):
    def __init__(self, inp: int, out: int, kind: str = "mlp", merge: int = 1):
        super().__init__()
        if kind not in ("linear", "mlp"):
            raise ValueError("a projector is linear or mlp")
        self.merge = merge
        inp = inp * merge * merge
        self.norm = nn.LayerNorm(inp) if merge > 1 else None
        self.fc1 = nn.Linear(inp, out)
        self.fc2 = nn.Linear(out, out) if kind == "mlp" else None

    def forward(self, feats: torch.Tensor) -> torch.Tensor:
        """``[B, N, d]`` patch features on a square grid -> ``[B, N / merge^2, out]``."""
        if self.merge > 1:
            B, N, d = feats.shape
            g = int(math.isqrt(N))
            if g * g != N or g % self.merge:
                raise ValueError(f"{N} patches do not fold by {self.merge}")
            m = self.merge
            feats = feats.reshape(B, g // m, m, g // m, m, d).permute(0, 1, 3, 2, 4, 5).reshape(B, (g // m) ** 2, m * m * d)
            feats = self.norm(feats)
        h = self.fc1(feats)
        return h if self.fc2 is None else self.fc2(F.gelu(h))


def expand_placeholders(tokens: Sequence[int], placeholder: int, count: int) -> List[int]:
    out: List[int] = []
    for t in tokens:
        out.extend([placeholder] * count if t == placeholder else [t])
    return out


def splice(embeddings: torch.Tensor, tokens: torch.Tensor, placeholder: int, features: torch.Tensor) -> torch.Tensor:
    """Write ``features [M, d]`` (every item's tokens, in batch order) over the positions of ``tokens`` that hold ``placeholder``."""
    at = tokens == placeholder
    n = int(at.sum())
    if n != features.shape[0]:
        raise ValueError(f"the rows hold {n} placeholder tokens for {features.shape[0]} feature vectors: expand each placeholder to one per patch")
    out = embeddings.clone()
    out[at] = features.to(out.dtype)
    return out


class VisionLanguageModel(nn.Module):
    def __init__(self, vision: nn.Module, decoder: nn.Module, image_token_id: int, vision_features: int, projector: str = "mlp", merge: int = 1,
                 drop_class_token: bool = True, freeze_vision: bool = True, feature_layer: Optional[int] = None):
        super().__init__()
        self.vision, self.decoder, self.image_token_id = vision, decoder, image_token_id
        self.projector = Projector(vision_features, decoder.config.emb_features, projector, merge)
        self.drop_class_token, self.feature_layer = drop_class_token, feature_layer
        if freeze_vision:
            for p in vision.parameters():
                p.requires_grad_(False)
        self.freeze_vision = freeze_vision
        self.config, self.vocab_size = decoder.config, decoder.vocab_size

    def image_features(self, images: torch.Tensor) -> torch.Tensor:
        """``[N, C, H, W]`` -> ``[N, tokens per image, d_decoder]``."""
        ctx = torch.no_grad() if self.freeze_vision else torch.enable_grad()
        with ctx:
            tokens, _ = self.vision(images, return_layer=self.feature_layer) if self.feature_layer is not None else self.vision(images)
        if self.drop_class_token and getattr(self.vision, "class_token", None) is not None:
            tokens = tokens[:, 1:]
        return self.projector(tokens)

    def tokens_per_image(self, image_size: int) -> int:
        n = (image_size // self.vision.patch) ** 2
        return n // (self.projector.merge ** 2)

    def embeddings(self, tokens: torch.Tensor, images: Optional[torch.Tensor]) -> torch.Tensor:
        emb = self.decoder.embed(tokens)
        if images is None or images.numel() == 0:
            return emb
        feats = self.image_features(images)
        return splice(emb, tokens, self.image_token_id, feats.reshape(-1, feats.shape[-1]))

    def hidden(self, tokens, positions=None, segment_ids=None, cache=None, train: bool = False, images: Optional[torch.Tensor] = None, **kw):
        return self.decoder.hidden(tokens, positions, segment_ids, cache, train, embeddings=self.embeddings(tokens, images), **kw)

    def head_weight(self):
        return self.decoder.head_weight()

    @property
    def head(self):
        return self.decoder.head

    @property
    def head_parameter(self) -> str:
        """The name of the output table among this module's parameters (what a chunked-loss objective looks up in a variable tree)."""
        return "decoder.embed.weight" if self.decoder.head is None else "decoder.head.weight"

    def logits(self, hidden):
        return self.decoder.logits(hidden)

    def forward(self, tokens, images: Optional[torch.Tensor] = None, return_hidden: bool = False, **kw):
        h = self.hidden(tokens, images=images, **kw)
        return h if return_hidden else self.decoder.logits(h)


# ------------------------------------------------------------------------------------------------ audio
def mel_filters(sample_rate: int, n_fft: int, n_mels: int) -> torch.Tensor:
    """Triangular filters on the mel scale (Slaney's: linear below 1 kHz, logarithmic above), area-normalised: ``[n_mels, n_fft / 2 + 1]``."""
    def hz_to_mel(f):
        f = torch.as_tensor(f, dtype=torch.float64)
        return torch.where(f < 1000.0, f / (200.0 / 3), 15.0 + torch.log(f.clamp_min(1e-9) / 1000.0) / (math.log(6.4) / 27.0))

    def mel_to_hz(m):
        return torch.where(m < 15.0, m * (200.0 / 3), 1000.0 * torch.exp((m - 15.0) * (math.log(6.4) / 27.0)))
    freqs = torch.linspace(0, sample_rate / 2, n_fft // 2 + 1, dtype=torch.float64)
    mels = torch.linspace(float(hz_to_mel(0.0)), float(hz_to_mel(sample_rate / 2)), n_mels + 2, dtype=torch.float64)
    hz = mel_to_hz(mels)
    lower, centre, upper = hz[:-2, None], hz[1:-1, None], hz[2:, None]
    up = (freqs[None] - lower) / (centre - lower)
    down = (upper - freqs[None]) / (upper - centre)
    bank = torch.clamp(torch.minimum(up, down), min=0.0)
    return (bank * (2.0 / (upper - lower))).float()


def log_mel(wave: torch.Tensor, sample_rate: int = 16000, n_fft: int = 400, hop: int = 160, n_mels: int = 80) -> torch.Tensor:
    """``[B, samples]`` -> ``[B, frames, n_mels]``: power spectrogram through the mel bank, ``log10`` clamped to 8 decades below the
    clip's maximum, then ``(x + 4) / 4``."""
    window = torch.hann_window(n_fft, device=wave.device)
    spec = torch.stft(wave.float(), n_fft, hop, window=window, return_complex=True)[..., :-1].abs() ** 2
    mel = mel_filters(sample_rate, n_fft, n_mels).to(wave.device) @ spec
    log = torch.log10(mel.clamp_min(1e-10))
    log = torch.maximum(log, log.amax((1, 2), keepdim=True) - 8.0)
    return ((log + 4.0) / 4.0).transpose(1, 2)


class AudioEncoder(nn.Module):
    def __init__(self, n_mels: int = 80, features: int = 256, layers: int = 4, heads: int = 4, max_frames: int = 1500):
        super().__init__()
        self.conv1 = nn.Conv1d(n_mels, features, 3, padding=1)
        self.conv2 = nn.Conv1d(features, features, 3, stride=2, padding=1)
        self.register_buffer("position", _sinusoids(max_frames, features), persistent=False)
        self.encoder = TransformerEncoder(EncoderConfig(features=features, layers=layers, heads=heads, mlp_features=4 * features))
        self.norm = nn.LayerNorm(features)
        self.features = features

    def frames(self, mel_frames: int) -> int:
        return (mel_frames + 1) // 2

    def forward(self, mel: torch.Tensor, lengths: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """``mel [B, frames, n_mels]`` -> (``[B, frames / 2, d]``, the mask of real output frames when ``lengths`` is given)."""
        if lengths is not None:                                             # padding frames read as silence, whatever they hold
            mel = mel * (torch.arange(mel.shape[1], device=mel.device)[None] < lengths[:, None])[..., None].to(mel.dtype)
        x = F.gelu(self.conv1(mel.transpose(1, 2)))
        x = F.gelu(self.conv2(x)).transpose(1, 2)
        x = x + self.position[: x.shape[1]].to(x.dtype)
        mask = None
        if lengths is not None:
            mask = torch.arange(x.shape[1], device=x.device)[None] < ((lengths + 1) // 2)[:, None]
        return self.norm(self.encoder(x, key_mask=mask)), mask


def _sinusoids(length: int, channels: int, max_timescale: float = 10000.0) -> torch.Tensor:
    inc = math.log(max_timescale) / (channels // 2 - 1)
    scaled = torch.arange(length)[:, None] * torch.exp(-inc * torch.arange(channels // 2))[None]
    return torch.cat([torch.sin(scaled), torch.cos(scaled)], 1)
