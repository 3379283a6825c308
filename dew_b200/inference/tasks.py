"""Inference tasks: what ``pipeline(...)`` / ``objective.pipeline(state)`` return.

``TextGeneration(prompts, max_new_tokens, key=, n=) -> Generation`` with ``.text, .lengths, .terminated``;
``task.bind(variables)`` swaps weights; ``task.quantized(...)`` returns a task over quantised weights
(reference: docs/concepts/inference.md:1-140; src/dew/inference/tasks.py).
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any, Optional, Sequence

import torch

from ..nn.kv_cache import KVCache
from ..sampling.text import Generation, Sampling, generate


@dataclass
class TextGeneration:
    model: torch.nn.Module
    variables: Any = None
    tokenizer: Any = None
    sampling: Sampling = field(default_factory=lambda: Sampling(temperature=0.0))
    kv_cache: Optional[KVCache] = None

    def __call__(self, prompts: Sequence[Any], max_new_tokens: int = 32, key: int = 0, n: int = 1,
                 sampling: Optional[Sampling] = None, strategy=None) -> Generation:
        return generate(self.model, self.variables, prompts, max_new_tokens, key=key, sampling=sampling or self.sampling,
                        n=n, tokenizer=self.tokenizer, kv_cache=self.kv_cache, strategy=strategy)

    def bind(self, variables) -> "TextGeneration":
        return replace(self, variables=variables)

    def quantized(self, quantization) -> "TextGeneration":
        from ..nn.quantization import quantize_variables
        from ..utils.trees import module_variables
        src = self.variables if self.variables is not None else module_variables(self.model)
        return replace(self, variables=quantize_variables(src, quantization))

    def offloaded(self, slots: int = 2) -> "TextGeneration":
        """Keep the decoder layers' weights in pinned host memory and stream them through ``slots`` device-resident copies
        while generating (``dew_b200.inference.banks.HostBanks``): for models larger than the GPU.  Bound variables are
        written into the module first, since the banks read the module's own parameters."""
        from .banks import HostBanks
        if self.variables is not None:
            from ..utils.trees import variables_for_call
            with torch.no_grad():
                for n, v in variables_for_call(self.model, self.variables).items():
                    if n in dict(self.model.named_parameters()):
                        self.model.get_parameter(n).copy_(v)
        dev = next(self.model.parameters()).device
        new = replace(self, variables=None)
        new.banks = self.banks = HostBanks(self.model.layers, dev, slots)      # both tasks share the one module, so both name its banks
        return new

    def score(self, tokens: torch.Tensor) -> torch.Tensor:
        """Per-token log-probabilities ``[B, S-1]`` of ``tokens`` under the model."""
        with torch.no_grad():
            logits = self.model(tokens[:, :-1]).float()
        return torch.log_softmax(logits, -1).gather(-1, tokens[:, 1:, None]).squeeze(-1)


def pipeline(source, *, mesh=None, layout=None, dtype=None, param_dtype=None, ema: Optional[bool] = None, step: Optional[int] = None,
             model=None, tokenizer=None, device=None):
    """Build a task from a checkpoint directory (``run.json`` names the model), a ``TrainState`` + model, or a module."""
    import os
    from ..checkpoints import Checkpoints
    from ..utils.registry import lookup
    if isinstance(source, (str, os.PathLike)):
        ck = Checkpoints(source)
        run = ck.read_run() or {}
        if model is None:
            if "model" not in run:
                raise FileNotFoundError(f"{source}/run.json does not describe a model; pass model=")
            model = lookup(run["model"]["name"])(**run["model"].get("fields", {}))
        if tokenizer is None and run.get("tokenizer") == "byte":
            from ..data import ByteTokenizer
            tokenizer = ByteTokenizer()
        from ..checkpoints.state_trees import leaf_kinds
        ck.kinds = leaf_kinds(model)
        variables = ck.variables(step=step, ema=ema, param_dtype=param_dtype or dtype, device=device or "cpu")
        if device is not None:
            model = model.to(device)
        if dtype is not None:
            model = model.to(dtype)
        return TextGeneration(model, variables, tokenizer)
    if isinstance(source, torch.nn.Module):
        return TextGeneration(source, None, tokenizer)
    raise TypeError(f"cannot build a pipeline from {type(source).__name__}")
