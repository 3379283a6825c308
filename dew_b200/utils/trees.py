"""Nested-dict "variable trees" and their flat path form.

A variable tree is a plain nested ``dict`` whose leaves are tensors (or ``None``).  The flat
form keys every leaf by its ``/``-joined path, e.g. ``params/layers_0/attn/q_proj/kernel``; the
same paths name leaves in checkpoints (reference layout: src/dew/checkpoints/_payloads.py:1-60).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Iterator, Mapping, Tuple

import torch

SEP = "/"


def flatten(tree: Mapping[str, Any], prefix: str = "") -> Dict[str, Any]:
    """Flat ``path -> leaf`` mapping of a nested dict, in insertion order."""
    flat: Dict[str, Any] = {}
    for name, value in tree.items():
        path = f"{prefix}{SEP}{name}" if prefix else str(name)
        if isinstance(value, Mapping):
            flat.update(flatten(value, path))
        else:
            flat[path] = value
    return flat


def unflatten(flat: Mapping[str, Any]) -> Dict[str, Any]:
    """Inverse of :func:`flatten`."""
    tree: Dict[str, Any] = {}
    for path, value in flat.items():
        node = tree
        parts = path.split(SEP)
        for part in parts[:-1]:
            node = node.setdefault(part, {})
        node[parts[-1]] = value
    return tree


def tree_map(fn: Callable[..., Any], tree: Any, *rest: Any) -> Any:
    """Apply ``fn`` leaf-wise over one or more trees of identical structure."""
    if isinstance(tree, Mapping):
        return {k: tree_map(fn, v, *(r[k] for r in rest)) for k, v in tree.items()}
    if isinstance(tree, (list, tuple)):
        mapped = [tree_map(fn, v, *(r[i] for r in rest)) for i, v in enumerate(tree)]
        return type(tree)(mapped) if not hasattr(tree, "_fields") else type(tree)(*mapped)
    return fn(tree, *rest)


def leaves(tree: Any) -> Iterator[Any]:
    if isinstance(tree, Mapping):
        for v in tree.values():
            yield from leaves(v)
    elif isinstance(tree, (list, tuple)):
        for v in tree:
            yield from leaves(v)
    else:
        yield tree


def tensor_leaves(tree: Any) -> Iterator[torch.Tensor]:
    for leaf in leaves(tree):
        if isinstance(leaf, torch.Tensor):
            yield leaf


def tree_bytes(tree: Any) -> int:
    return sum(t.numel() * t.element_size() for t in tensor_leaves(tree))


def tree_count(tree: Any) -> int:
    return sum(t.numel() for t in tensor_leaves(tree))


def module_path_to_tree_path(name: str) -> str:
    """``layers.0.attn.q_proj.weight`` -> ``layers_0/attn/q_proj/weight``.

    Integer components fold into the preceding name the way Flax names repeated sub-modules
    (``layers_0``), which keeps checkpoint paths stable across frameworks.
    """
    out = []
    for part in name.split("."):
        if part.isdigit() and out:
            out[-1] = f"{out[-1]}_{part}"
        else:
            out.append(part)
    return SEP.join(out)


def module_variables(module: torch.nn.Module) -> Dict[str, Any]:
    """The module's parameters as a ``{'params': tree}`` variable tree (leaves alias the module's own)."""
    flat = {module_path_to_tree_path(n): p for n, p in module.named_parameters()}
    buffers = {module_path_to_tree_path(n): b for n, b in module.named_buffers() if b is not None}
    tree: Dict[str, Any] = {"params": unflatten(flat)}
    if buffers:
        tree["buffers"] = unflatten(buffers)
    return tree


def variables_for_call(module: torch.nn.Module, variables: Mapping[str, Any]) -> Dict[str, torch.Tensor]:
    """Map a variable tree back to ``torch.func.functional_call`` names for ``module``."""
    flat_params = flatten(variables.get("params", {}))
    flat_buffers = flatten(variables.get("buffers", {})) if "buffers" in variables else {}
    out: Dict[str, torch.Tensor] = {}
    for n, _ in module.named_parameters():
        key = module_path_to_tree_path(n)
        if key in flat_params:
            out[n] = flat_params[key]
    for n, _ in module.named_buffers():
        key = module_path_to_tree_path(n)
        if key in flat_buffers:
            out[n] = flat_buffers[key]
    return out


def structure(tree: Any) -> Any:
    """Shapes and dtypes of a tree (a template for restore)."""
    return tree_map(lambda t: (tuple(t.shape), str(t.dtype)) if isinstance(t, torch.Tensor) else t, tree)


def same_structure(a: Any, b: Any) -> Tuple[bool, str]:
    fa, fb = flatten(a) if isinstance(a, Mapping) else {"": a}, flatten(b) if isinstance(b, Mapping) else {"": b}
    if fa.keys() != fb.keys():
        missing = sorted(set(fa) ^ set(fb))
        return False, f"paths differ: {missing[:8]}"
    for k in fa:
        x, y = fa[k], fb[k]
        if isinstance(x, torch.Tensor) and isinstance(y, torch.Tensor) and x.shape != y.shape:
            return False, f"{k}: {tuple(x.shape)} vs {tuple(y.shape)}"
    return True, ""
