"""The text-to-image task: a trained diffusion model that turns prompts (or other conditions) into images, beside
``TextGeneration``.  The reverse walk is ``dew_b200.sampling.walk_and_decode``.

``TextToImage.from_objective(objective, variables)`` takes process, inputs (condition encoders, null values), autoencoder,
solver, guidance and step count from a ``DiffusionObjective``; calling the task returns ``Images`` (``decoded`` in [-1, 1],
``pixels()`` uint8, ``pil()``).  ``ImageRequest`` is one queued request of a serving loop: requests that share settings
are walked together as one batch.

Reference: src/dew/inference/images.py (``Images`` :102, ``ImageSettings`` :144, ``TextToImage`` :175-824, ``ImageRequest`` :826).
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..sampling import CFG, DDIM, Guidance, Solver, walk_and_decode
from ..utils import keys as K


@dataclass
class Images:
    """A batch of generated images: ``decoded [B, H, W, C]`` floats in [-1, 1] (``latents`` when decoding was skipped)."""
    decoded: Optional[torch.Tensor]
    latents: Optional[torch.Tensor] = None

    def host(self) -> "Images":
        return Images(None if self.decoded is None else self.decoded.cpu(), None if self.latents is None else self.latents.cpu())

    def pixels(self) -> torch.Tensor:
        if self.decoded is None:
            raise ValueError("these images were not decoded (decode=False); decode the latents first")
        return ((self.decoded.float().clamp(-1, 1) + 1) * 127.5).round().to(torch.uint8)

    def pil(self) -> list:
        from PIL import Image
        return [Image.fromarray(p.cpu().numpy()) for p in self.pixels()]


@dataclass(frozen=True)
class ImageSettings:
    """What a request may set; None takes the task's own."""
    steps: Optional[int] = None
    guidance: Any = "task"              # a Guidance, a float (CFG scale), None (unguided) or "task"
    solver: Optional[Solver] = None
    height: Optional[int] = None
    width: Optional[int] = None
    decode: bool = True

    def __post_init__(self):
        if self.steps is not None and (type(self.steps) is not int or self.steps < 1):
            raise ValueError("steps must be a positive integer")


@dataclass
class TextToImage:
    model: torch.nn.Module
    process: Any
    inputs: Any                                       # InputSpec: conditions with encoders and null values
    variables: Any = None
    autoencoder: Any = None
    solver: Solver = field(default_factory=DDIM)
    guidance: Optional[Guidance] = field(default_factory=lambda: CFG(3.0))
    steps: int = 50
    sample_shape: Optional[Tuple[int, ...]] = None     # latent (H, W, C) the model denoises

    @classmethod
    def from_objective(cls, objective, variables=None) -> "TextToImage":
        shape = tuple(objective.inputs.sample.shape) or None
        return cls(objective.model, objective.process, objective.inputs, variables, objective.autoencoder, objective.solver,
                   objective.guidance, objective.steps, shape)

    def bind(self, variables) -> "TextToImage":
        return replace(self, variables=variables)

    def quantized(self, quantization) -> "TextToImage":
        from ..nn.quantization import quantize_variables
        from ..utils.trees import module_variables
        src = self.variables if self.variables is not None else module_variables(self.model)
        return replace(self, variables=quantize_variables(src, quantization))

    # ------------------------------------------------------------------ pieces
    def latent_shape(self, height: Optional[int] = None, width: Optional[int] = None) -> Tuple[int, ...]:
        if self.sample_shape is None:
            raise ValueError("the task does not know its sample shape; pass sample_shape=(H, W, C)")
        H, W, C = self.sample_shape
        if height is None and width is None:
            return (H, W, C)
        factor = getattr(self.autoencoder, "downscale", 1) if self.autoencoder is not None else 1
        h, w = (height or H * factor), (width or W * factor)
        if h % factor or w % factor:
            raise ValueError(f"height and width must be multiples of the autoencoder's factor {factor}")
        return (h // factor, w // factor, C)

    def encode(self, conditions: Mapping[str, Any], rows: int) -> Dict[str, torch.Tensor]:
        """Run each given condition through its encoder (prompts -> text features, labels -> ids ...)."""
        out = {}
        for name, value in conditions.items():
            if name not in self.inputs.conditions:
                raise KeyError(f"the model has no condition {name!r}; it has {sorted(self.inputs.conditions)}")
            cond = self.inputs.conditions[name]
            if cond.tokenizer is not None and isinstance(value, (list, tuple)) and value and isinstance(value[0], str):
                value = cond.tokenizer(list(value))
            v = cond.encoder(value) if cond.encoder is not None else torch.as_tensor(value)
            if v.shape[0] != rows:
                raise ValueError(f"condition {name!r} has {v.shape[0]} rows for {rows} images")
            out[name] = v
        return out

    def unconditional(self, given: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        out = {}
        for name, v in given.items():
            null = self.inputs.conditions[name].null
            out[name] = torch.zeros_like(v) if null is None else torch.as_tensor(null).to(v).expand_as(v)
        return out

    def _guidance(self, guidance):
        if isinstance(guidance, str) and guidance == "task":
            return self.guidance
        if guidance is None or isinstance(guidance, Guidance):
            return guidance
        return CFG(float(guidance))

    # ------------------------------------------------------------------ the call
    @torch.no_grad()
    def __call__(self, prompts: Optional[Sequence[str]] = None, *, conditions: Optional[Mapping[str, Any]] = None, n: Optional[int] = None,
                 key=0, settings: Optional[ImageSettings] = None, on_step: Optional[Callable[[int, torch.Tensor], None]] = None,
                 **overrides) -> Images:
        """``prompts`` fill the condition named "text"; other conditions by name.  ``n`` images when nothing conditions the
        model.  ``on_step(i, x)`` sees the state after every solver step."""
        s = settings or ImageSettings(**overrides)
        given_raw = dict(conditions or {})
        if prompts is not None:
            given_raw["text"] = list(prompts)
        rows = n if n is not None else (len(next(iter(given_raw.values()))) if given_raw else 1)
        given = self.encode(given_raw, rows)
        dev = next(self.model.parameters()).device
        given = {k: v.to(dev) for k, v in given.items()}
        den = self.process.denoiser(self.model, self.variables, given)
        g = self._guidance(s.guidance) if given else None
        shape = (rows, *self.latent_shape(s.height, s.width))
        x_T = self.process.noise(K.fold_in(K.key(key), "prior"), shape).to(dev)
        record = (lambda x, state, denoised: on_step(len(seen) or 0, x) or seen.append(0)) if on_step is not None else None
        seen: List[int] = []
        out = walk_and_decode(den, x_T, s.steps or self.steps, solver=s.solver or self.solver, guidance=g, key=key,
                              null_conditions=self.unconditional(given) if g is not None else None, record=record,
                              autoencoder=None, clip=None)
        latents = out[0] if record is not None else out
        if not s.decode:
            return Images(None, latents)
        decoded = self.autoencoder.decode(latents) if self.autoencoder is not None else latents
        return Images(decoded.clamp(-1, 1), latents)


@dataclass
class ImageRequest:
    """One queued request: prompts / conditions, its own key and settings."""
    prompts: Optional[Sequence[str]] = None
    conditions: Optional[Mapping[str, Any]] = None
    n: Optional[int] = None
    key: int = 0
    settings: ImageSettings = field(default_factory=ImageSettings)


def serve(task: TextToImage, requests: Sequence[ImageRequest]) -> List[Images]:
    """Answer ``requests`` in order.  Each request is its own walk (its own key and prior draw), so a request's images do
    not depend on what else is queued."""
    return [task(r.prompts, conditions=r.conditions, n=r.n, key=r.key, settings=r.settings) for r in requests]
