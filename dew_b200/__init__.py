"""dew_b200: a Blackwell-native (sm_100a) training and serving framework with the capabilities of Dew.

One facade, lazily bound (importing the package imports no CUDA library and allocates nothing):
``Trainer, TrainState, Step, Aux, EMASpec, MeshSpec, Layout, Checkpoints, Tracker (+ Wandb / Local / MLflow /
TensorBoard / Trackers), Evaluation, ProfileWindow, Objective, Supervised, Dataset, Process, Mean, InputSpec, Field,
Condition, sample, CFG, pipeline, Profiler, gpu_facts, kernels, ImageGrid / VideoGrid / TextSamples /
Representations / TokenScores, register, Best / Keep / Plateau`` (reference facade: src/dew/__init__.py:120-145).
"""
from __future__ import annotations

import importlib
from typing import Any

__version__ = "0.1.0"

_EXPORTS = {
    "Trainer": "training", "TrainState": "training", "Cooldown": "training", "Best": "training", "Plateau": "training", "Pause": "training",
    "Evaluation": "training", "ProfileWindow": "training", "Tracker": "training", "LocalTracker": "training",
    "WandbTracker": "training", "Wandb": "training", "MLflowTracker": "training", "TensorBoardTracker": "training",
    "Trackers": "training", "MemoryTracker": "training", "ConsoleTracker": "training",
    "Step": "objectives", "Aux": "objectives", "EMASpec": "objectives", "Objective": "objectives", "Mean": "objectives",
    "Ratio": "objectives", "Moments": "objectives", "Supervised": "objectives", "DiffusionObjective": "objectives",
    "LMObjective": "objectives", "JepaObjective": "objectives",
    "MeshSpec": "parallel.mesh", "Layout": "parallel.layout",
    "Checkpoints": "checkpoints", "CorruptCheckpoint": "checkpoints", "Keep": "checkpoints", "Ranking": "checkpoints",
    "Dataset": "data", "Memory": "data", "Loader": "data", "TokenFiles": "data", "ByteTokenizer": "data",
    "Process": "diffusion", "EDM": "diffusion", "Flow": "diffusion", "Karras": "diffusion",
    "InputSpec": "inputs", "Field": "inputs", "Condition": "inputs", "unit_range": "inputs",
    "sample": "sampling", "CFG": "sampling", "Heun": "sampling", "DDIM": "sampling", "Euler": "sampling",
    "OptimConfig": "optim",
    "pipeline": "inference", "Server": "inference", "KVCache": "nn.kv_cache",
    "Profiler": "telemetry", "gpu_facts": "utils.devices", "GpuFacts": "utils.devices",
    "ImageGrid": "utils.artifacts", "VideoGrid": "utils.artifacts", "TextSamples": "utils.artifacts",
    "Representations": "utils.artifacts", "TokenScores": "utils.artifacts",
    "register": "utils.registry",
    "SimpleDiT": "models", "CausalTransformer": "models", "generate": "sampling.text", "Sampling": "sampling.text",
}

__all__ = sorted(_EXPORTS) + ["kernels", "ops"]


def __getattr__(name: str) -> Any:
    if name == "kernels" or name == "ops":
        return importlib.import_module(".ops", __name__)
    if name in _EXPORTS:
        return getattr(importlib.import_module(f".{_EXPORTS[name]}", __name__), name)
    raise AttributeError(f"module 'dew_b200' has no attribute {name!r}")
