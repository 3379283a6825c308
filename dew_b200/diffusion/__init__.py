from . import presets, schedules, transforms
from .presets import EDM, Cosine, CosineContinuous, Exp, Flow, JiT, Karras, Linear, MeanFlow, ResolutionShift, Shortcut, Sqrt
from .process import Denoiser, Process

__all__ = ["JiT", "MeanFlow", "Shortcut", "EDM", "Karras", "Cosine", "CosineContinuous", "Linear", "Exp", "Sqrt", "Flow", "ResolutionShift",
           "Process", "Denoiser", "presets", "schedules", "transforms"]
