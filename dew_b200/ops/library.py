"""ctypes binding to ``libdewb.so`` (the sm_100a kernels) and the device status word.

The library is built in-tree by :mod:`dew_b200.ops.build`.  On a machine with a GPU every op in
:mod:`dew_b200.ops` runs through it; if it is missing there the ops raise instead of silently falling back,
so a GPU test can never pass on an eager path by accident.  On a CPU-only machine the ops use their
PyTorch reference implementations and this module is never loaded.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path
from typing import Dict, Optional

import torch

_LIB: Optional[ctypes.CDLL] = None
_LIB_PATH = Path(__file__).resolve().parent / "libdewb.so"
_STATUS: Dict[int, torch.Tensor] = {}

ERROR_NAMES = {0: "ok", 1: "wait for a TMA stage timed out", 2: "wait for a free stage timed out",
               3: "wait for an accumulator timed out", 4: "wait for a drained accumulator timed out",
               5: "wait for a peer's flag timed out", 6: "bad argument", 7: "wait timed out"}


class KernelError(RuntimeError):
    """A launcher refused its arguments or a kernel reported a timed-out wait."""


class LibraryMissing(RuntimeError):
    pass


def path() -> Path:
    return _LIB_PATH


def exists() -> bool:
    return _LIB_PATH.exists()


def load(build_if_missing: bool = False) -> ctypes.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    if not _LIB_PATH.exists():
        if build_if_missing:
            from . import build
            build.build(verbose=False)
        else:
            raise LibraryMissing(f"{_LIB_PATH} is not built; run `python -m dew_b200.ops.build`")
    _LIB = ctypes.CDLL(str(_LIB_PATH))
    return _LIB


def use_cuda(*tensors: torch.Tensor) -> bool:
    """True when the op must run on the CUDA library (all tensors on a GPU)."""
    t = next((x for x in tensors if isinstance(x, torch.Tensor)), None)
    if t is None or not t.is_cuda:
        return False
    if os.environ.get("DEWB_FORCE_REFERENCE") == "1":
        return False
    load()  # raises LibraryMissing on a GPU box without the build
    ensure_device(t)
    return True


_TLS = threading.local()


def ensure_device(t: torch.Tensor) -> None:
    """Make ``t``'s device current for the library's own CUDA runtime on this thread (autograd runs backward on
    worker threads where nothing has selected a device yet)."""
    idx = t.device.index if t.device.index is not None else torch.cuda.current_device()
    if getattr(_TLS, "device", None) != idx:
        check(load().dewb_set_device(ctypes.c_int(idx)), "set_device")
        _TLS.device = idx


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def status(device: Optional[torch.device] = None) -> torch.Tensor:
    """The per-device int32 status word kernels write a non-zero code into when a bounded wait gives up."""
    idx = torch.cuda.current_device() if device is None else (device.index or 0)
    if idx not in _STATUS:
        _STATUS[idx] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
    return _STATUS[idx]


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronising read of the status word; raises if any kernel reported an error since the last check."""
    word = status(device)
    code = int(word.item())
    if code != 0:
        word.zero_()
        raise KernelError(f"device kernel reported: {ERROR_NAMES.get(code, code)}")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what}: launcher returned {rc}")


LAUNCHES = 0


def count_launches(n: int = 1) -> None:
    """Bookkeeping of how many of this library's kernels were launched (bench.py reports it)."""
    global LAUNCHES
    LAUNCHES += n
