from . import presets, schedules, transforms
from .presets import EDM, Cosine, CosineContinuous, Exp, Flow, Karras, Linear, ResolutionShift, Sqrt
from .process import Denoiser, Process

__all__ = ["EDM", "Karras", "Cosine", "CosineContinuous", "Linear", "Exp", "Sqrt", "Flow", "ResolutionShift",
           "Process", "Denoiser", "presets", "schedules", "transforms"]
