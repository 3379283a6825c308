"""Push a new policy version from a trainer GPU into inference replicas by NCCL broadcast, driving ``libnccl`` directly
through ``ctypes`` on a communicator of its own (the one place this library calls NCCL without ``torch.distributed``:
the receiving engine is another program, so the group is opened from a shared unique id, not from a process group).

Protocol (rank 0 = the trainer, ranks 1.. = the engine's workers): the trainer mints the unique id and hands it to the
engine out of band (base64); both sides enter ``ncclCommInitRankConfig`` (non-blocking on this side, so a peer that
never comes is noticed by the ``watch`` callback and the group is aborted rather than waited on); a one-element
all-reduce warms the group up; then every tensor is broadcast from rank 0 in the order of ``names``, in pieces of at
most ``CHUNK_BYTES``.  ``Collectives`` is the seam a fake stands behind in CPU tests.

Reference: src/dew/inference/nccl.py:82-470 (``Collectives`` protocol, ``_Library``, ``NCCLPush``).
"""
from __future__ import annotations

import base64
import ctypes
import glob
import os
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Mapping, Optional, Protocol, Sequence

import torch

CHUNK_BYTES = 512 << 20
# ncclDataType_t codes (nccl.h, stable since 2.27: the first release with the FP8 codes)
DTYPES = {torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4, torch.float16: 6, torch.float32: 7,
          torch.float64: 8, torch.bfloat16: 9, torch.float8_e4m3fn: 10}
NCCL_SUM = 0
NCCL_SUCCESS, NCCL_IN_PROGRESS = 0, 7


class UniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 128)]

    def b64(self) -> str:
        return base64.b64encode(bytes(self.internal)).decode()

    @classmethod
    def from_b64(cls, text: str) -> "UniqueId":
        raw = base64.b64decode(text)
        uid = cls()
        ctypes.memmove(uid.internal, raw, 128)
        return uid


class _Config(ctypes.Structure):
    """``ncclConfig_t`` up to the fields this module sets; the initialiser macro's magic / version head the struct and
    every other field keeps its "undefined" sentinel (INT_MIN / null)."""
    _fields_ = [("size", ctypes.c_size_t), ("magic", ctypes.c_uint), ("version", ctypes.c_uint), ("blocking", ctypes.c_int),
                ("cgaClusterSize", ctypes.c_int), ("minCTAs", ctypes.c_int), ("maxCTAs", ctypes.c_int),
                ("netName", ctypes.c_char_p), ("splitShare", ctypes.c_int), ("trafficClass", ctypes.c_int),
                ("commName", ctypes.c_char_p), ("collnetEnable", ctypes.c_int), ("CTAPolicy", ctypes.c_int),
                ("shrinkShare", ctypes.c_int), ("nvlsCTAs", ctypes.c_int), ("nChannelsPerNetPeer", ctypes.c_int),
                ("nvlinkCentricSched", ctypes.c_int), ("pad", ctypes.c_int * 16)]


class Collectives(Protocol):
    def unique_id(self) -> UniqueId: ...
    def open(self, uid: UniqueId, rank: int, world: int, watch: Optional[Callable[[], None]] = None) -> object: ...
    def all_reduce(self, comm, tensor: torch.Tensor) -> None: ...
    def broadcast(self, comm, tensor: torch.Tensor, root: int = 0) -> None: ...
    def settled(self, comm, watch: Optional[Callable[[], None]] = None) -> None: ...
    def abort(self, comm) -> None: ...


class PushFailed(RuntimeError):
    pass


def find_library() -> str:
    """The NCCL the engine is most likely to run: the wheel beside torch, else the system one."""
    import importlib.util
    spec = importlib.util.find_spec("nvidia.nccl")
    if spec is not None and spec.submodule_search_locations:
        hits = glob.glob(os.path.join(list(spec.submodule_search_locations)[0], "lib", "libnccl.so*"))
        if hits:
            return sorted(hits)[0]
    return "libnccl.so.2"


class NcclLibrary:
    """``Collectives`` over a real ``libnccl`` (the library's version must equal the engine's: NCCL refuses a peer of
    another version when the group opens)."""

    def __init__(self, library: Optional[str] = None, device: Optional[torch.device] = None, timeout_s: float = 120.0):
        self.lib = ctypes.CDLL(library or find_library())
        self.device = torch.device(device if device is not None else ("cuda", torch.cuda.current_device()))
        self.timeout_s = timeout_s
        v = ctypes.c_int()
        self._ok(self.lib.ncclGetVersion(ctypes.byref(v)))
        self.version = v.value

    def _ok(self, status: int) -> None:
        if status not in (NCCL_SUCCESS, NCCL_IN_PROGRESS):
            self.lib.ncclGetErrorString.restype = ctypes.c_char_p
            raise PushFailed(f"NCCL error {status}: {self.lib.ncclGetErrorString(status).decode()}")

    def unique_id(self) -> UniqueId:
        uid = UniqueId()
        self._ok(self.lib.ncclGetUniqueId(ctypes.byref(uid)))
        return uid

    def _config(self) -> _Config:
        cfg = _Config()
        cfg.size, cfg.magic, cfg.version = ctypes.sizeof(_Config), 0xcafebeef, self.version
        undefined = -2 ** 31
        for name, kind in _Config._fields_[3:-1]:
            setattr(cfg, name, None if kind is ctypes.c_char_p else undefined)
        cfg.blocking = 0
        return cfg

    def open(self, uid: UniqueId, rank: int, world: int, watch=None):
        comm = ctypes.c_void_p()
        cfg = self._config()
        with torch.cuda.device(self.device):
            self._ok(self.lib.ncclCommInitRankConfig(ctypes.byref(comm), world, uid, rank, ctypes.byref(cfg)))
        self.settled(comm, watch)
        return comm

    def _stream(self) -> ctypes.c_void_p:
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def all_reduce(self, comm, tensor: torch.Tensor) -> None:
        self._ok(self.lib.ncclAllReduce(ctypes.c_void_p(tensor.data_ptr()), ctypes.c_void_p(tensor.data_ptr()),
                                        ctypes.c_size_t(tensor.numel()), DTYPES[tensor.dtype], NCCL_SUM, comm, self._stream()))

    def broadcast(self, comm, tensor: torch.Tensor, root: int = 0) -> None:
        self._ok(self.lib.ncclBroadcast(ctypes.c_void_p(tensor.data_ptr()), ctypes.c_void_p(tensor.data_ptr()),
                                        ctypes.c_size_t(tensor.numel()), DTYPES[tensor.dtype], root, comm, self._stream()))

    def settled(self, comm, watch=None) -> None:
        """Wait (bounded) until the communicator's pending call has finished and its stream is idle; ``watch`` is polled
        meanwhile and may raise to give up on a peer."""
        state, t0 = ctypes.c_int(NCCL_IN_PROGRESS), time.monotonic()
        while True:
            self._ok(self.lib.ncclCommGetAsyncError(comm, ctypes.byref(state)))
            if state.value == NCCL_SUCCESS and torch.cuda.current_stream(self.device).query():
                return
            if state.value not in (NCCL_SUCCESS, NCCL_IN_PROGRESS):
                raise PushFailed(f"NCCL async error {state.value}")
            if watch is not None:
                watch()
            if time.monotonic() - t0 > self.timeout_s:
                raise PushFailed(f"NCCL call still in progress after {self.timeout_s} s")
            time.sleep(0.002)

    def abort(self, comm) -> None:
        self.lib.ncclCommAbort(comm)


def chunks(tensor: torch.Tensor, limit: int = CHUNK_BYTES) -> List[torch.Tensor]:
    flat = tensor.reshape(-1)
    per = max(1, limit // tensor.element_size())
    return [flat[i:i + per] for i in range(0, flat.numel(), per)] or [flat]


@dataclass
class NCCLPush:
    """``push(tensors, version)`` broadcasts ``tensors`` (name -> device tensor, the exported checkpoint layout) from
    this process (rank 0) into ``receivers`` engine ranks.

    ``announce(uid_b64, names, shapes, dtypes, version)`` tells the engine what is coming (for vLLM: the HTTP calls that
    start the update and list the tensors) and is called before the group opens; ``finish(version)`` after the last
    tensor has landed; ``watch()`` is polled while waiting and raises if the engine reported a failure."""
    receivers: int
    collectives: Collectives
    announce: Callable[..., None]
    finish: Callable[[int], None] = lambda version: None
    watch: Optional[Callable[[], None]] = None
    chunk_bytes: int = CHUNK_BYTES
    comm: object = field(default=None, init=False)
    pushed: List[int] = field(default_factory=list, init=False)

    def _open(self, names, tensors, version) -> None:
        uid = self.collectives.unique_id()
        self.announce(uid.b64(), list(names), [tuple(tensors[n].shape) for n in names],
                      [str(tensors[n].dtype).replace("torch.", "") for n in names], version)
        self.comm = self.collectives.open(uid, 0, 1 + self.receivers, self.watch)
        warm = torch.ones(1, dtype=torch.float32, device=next(iter(tensors.values())).device)
        self.collectives.all_reduce(self.comm, warm)
        self.collectives.settled(self.comm, self.watch)

    def push(self, tensors: Mapping[str, torch.Tensor], version: int, names: Optional[Sequence[str]] = None) -> None:
        names = list(names) if names is not None else sorted(tensors)
        try:
            if self.comm is None:
                self._open(names, tensors, version)
            else:
                self.announce(None, names, [tuple(tensors[n].shape) for n in names],
                              [str(tensors[n].dtype).replace("torch.", "") for n in names], version)
            for n in names:
                t = tensors[n]
                if t.dtype not in DTYPES:
                    raise PushFailed(f"{n}: dtype {t.dtype} has no NCCL code")
                for piece in chunks(t.contiguous(), self.chunk_bytes):
                    self.collectives.broadcast(self.comm, piece, 0)
                self.collectives.settled(self.comm, self.watch)
            self.finish(version)
            self.pushed.append(version)
        except Exception:
            self.close(abort=True)
            raise

    def close(self, abort: bool = False) -> None:
        if self.comm is not None:
            self.collectives.abort(self.comm)
            self.comm = None


class FakeCollectives:
    """In-memory stand-in: records the calls and, for ``broadcast``, copies rank 0's data into the receivers' tensors
    registered under the same call index - enough to test ordering, chunking and failure handling on CPU."""

    def __init__(self, fail_at: Optional[int] = None):
        self.calls: List[tuple] = []
        self.received: List[torch.Tensor] = []
        self.fail_at, self.aborted = fail_at, False

    def unique_id(self) -> UniqueId:
        uid = UniqueId()
        for i in range(128):
            uid.internal[i] = (i * 7) % 120
        return uid

    def open(self, uid, rank, world, watch=None):
        self.calls.append(("open", rank, world))
        return object()

    def all_reduce(self, comm, tensor):
        self.calls.append(("all_reduce", tensor.numel()))

    def broadcast(self, comm, tensor, root=0):
        if self.fail_at is not None and len(self.received) == self.fail_at:
            raise PushFailed("injected broadcast failure")
        self.calls.append(("broadcast", tensor.numel(), str(tensor.dtype)))
        self.received.append(tensor.clone())

    def settled(self, comm, watch=None):
        if watch is not None:
            watch()

    def abort(self, comm):
        self.aborted = True
