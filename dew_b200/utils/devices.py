"""What this library's kernels read of a GPU: a read-only ``GpuFacts`` record from the B200 table, refined by what the
CUDA driver reports of the device a process is placed on (queried through ``ctypes`` on ``libcuda``: no torch call, so
it also works before a context exists), and by measured peaks where a peaks file is given.

Reference: src/dew/nn/kernels/generation.py:1337-1395 (``GpuFacts`` / ``gpu_facts``), src/dew/_devices.py:434-460
(driver attribute queries).
"""
from __future__ import annotations

import ctypes
import dataclasses
import json
import os
from types import MappingProxyType
from typing import Mapping, Optional, Tuple

# CUdevice_attribute values (public driver API enum)
_ATTR = {"multiprocessors": 16, "clock_khz": 13, "l2_bytes": 38, "shared_optin": 97, "registers": 82, "resident_threads": 39,
         "resident_blocks": 106, "cc_major": 75, "cc_minor": 76, "memory_clock_khz": 36, "bus_width": 37}


@dataclasses.dataclass(frozen=True)
class GpuFacts:
    part: str
    generation: str
    capability: Optional[Tuple[int, int]]
    multiprocessors: Optional[int]
    clock_hz: Optional[float]
    memory_bandwidth: Optional[float]
    l2_bytes: Optional[int]
    shared_per_block: int
    registers: Optional[int]
    thread_registers: Optional[int]
    resident_threads: Optional[int]
    resident_blocks: Optional[int]
    tensor_memory_bytes: Optional[int]
    dense_peaks: Mapping[str, float]
    measured: Mapping[str, float]
    instruction_families: Tuple[str, ...]
    nvlink_bytes_per_s: Optional[float]

    def roofline_seconds(self, flops: float = 0.0, bytes_moved: float = 0.0, dtype: str = "bf16", measured: bool = True) -> float:
        """The slower of the math time and the memory time for one launch."""
        peak = self.measured.get(f"{dtype}_flops") if measured else None
        peak = peak or self.dense_peaks.get(dtype)
        bw = (self.measured.get("hbm_bytes_per_s") if measured else None) or self.memory_bandwidth
        return max(flops / peak if peak else 0.0, bytes_moved / bw if bw else 0.0)


_TABLE = {
    "sm100": dict(part="NVIDIA B200", generation="sm100", capability=(10, 0), multiprocessors=148, clock_hz=1.965e9, memory_bandwidth=7.7e12,
                  l2_bytes=126 * 2 ** 20, shared_per_block=227 * 1024, registers=65536, thread_registers=255, resident_threads=2048, resident_blocks=32,
                  tensor_memory_bytes=256 * 1024, dense_peaks={"bf16": 2.25e15, "fp16": 2.25e15, "fp8": 4.5e15, "fp4": 9e15, "tf32": 1.1e15},
                  instruction_families=("tcgen05", "mma.sync"), nvlink_bytes_per_s=900e9),
}
_ALIASES = {"b200": "sm100", "nvidia b200": "sm100", "sm_100a": "sm100", "sm100a": "sm100", "blackwell": "sm100"}


def _driver():
    try:
        lib = ctypes.CDLL("libcuda.so.1")
    except OSError:
        return None
    return lib if lib.cuInit(0) == 0 else None


def gpu_attribute(ordinal: int, name: str) -> Optional[int]:
    """One driver attribute of device ``ordinal`` (None with no driver / no such device)."""
    lib = _driver()
    if lib is None:
        return None
    dev, out = ctypes.c_int(), ctypes.c_int()
    if lib.cuDeviceGet(ctypes.byref(dev), ordinal) != 0:
        return None
    return out.value if lib.cuDeviceGetAttribute(ctypes.byref(out), _ATTR[name], dev) == 0 else None


def gpu_name(ordinal: int = 0) -> Optional[str]:
    lib = _driver()
    if lib is None:
        return None
    dev, buf = ctypes.c_int(), ctypes.create_string_buffer(128)
    if lib.cuDeviceGet(ctypes.byref(dev), ordinal) != 0 or lib.cuDeviceGetName(buf, 128, dev) != 0:
        return None
    return buf.value.decode()


def gpu_memory(ordinal: int = 0) -> Optional[int]:
    lib = _driver()
    if lib is None:
        return None
    dev, total = ctypes.c_int(), ctypes.c_size_t()
    if lib.cuDeviceGet(ctypes.byref(dev), ordinal) != 0 or lib.cuDeviceTotalMem_v2(ctypes.byref(total), dev) != 0:
        return None
    return total.value


def measured_peaks(path: Optional[str] = None) -> Mapping[str, float]:
    """Measured denominators from a peaks file (``hbm_gbs``, ``bf16_tflops``, ``bf16_tflops_sustained``), in SI units."""
    path = path or os.environ.get("DEWB_MEASURED_PEAKS") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        raw = json.load(open(path))
    except (OSError, ValueError):
        return {}
    out = {}
    if "hbm_gbs" in raw:
        out["hbm_bytes_per_s"] = float(raw["hbm_gbs"]) * 1e9
    if "bf16_tflops" in raw:
        out["bf16_flops"] = float(raw["bf16_tflops"]) * 1e12
    if "bf16_tflops_sustained" in raw:
        out["bf16_flops_sustained"] = float(raw["bf16_tflops_sustained"]) * 1e12
    return out


def gpu_facts(part: Optional[str] = None, ordinal: int = 0, peaks_file: Optional[str] = None) -> GpuFacts:
    """Facts of a named part ("b200", "sm100") or, with ``part`` None, of device ``ordinal`` as its driver reports it.
    Raises ``ValueError`` for a part this library knows nothing of, or when no GPU is present and none was named."""
    if part is not None:
        key = _ALIASES.get(part.lower(), part.lower())
        if key not in _TABLE:
            raise ValueError(f"no GPU named {part!r} is known; this library targets {sorted(_TABLE)}")
        row = dict(_TABLE[key])
    else:
        major, minor = gpu_attribute(ordinal, "cc_major"), gpu_attribute(ordinal, "cc_minor")
        if major is None:
            raise ValueError("no GPU is visible to the CUDA driver; name a part to read its facts")
        row = dict(_TABLE.get(f"sm{major}{minor}", _TABLE["sm100"] if major == 10 else {}))
        if not row:
            raise ValueError(f"device {ordinal} is compute capability {major}.{minor}; this library targets sm_100a")
        row["capability"] = (major, minor)
        row["part"] = gpu_name(ordinal) or row["part"]
        for field, attr, scale in (("multiprocessors", "multiprocessors", 1), ("clock_hz", "clock_khz", 1e3), ("l2_bytes", "l2_bytes", 1),
                                   ("shared_per_block", "shared_optin", 1), ("registers", "registers", 1), ("resident_threads", "resident_threads", 1),
                                   ("resident_blocks", "resident_blocks", 1)):
            v = gpu_attribute(ordinal, attr)
            if v:
                row[field] = type(row[field])(v * scale)
        mclk, width = gpu_attribute(ordinal, "memory_clock_khz"), gpu_attribute(ordinal, "bus_width")
        if mclk and width:
            row["memory_bandwidth"] = 2.0 * mclk * 1e3 * width / 8
    row["dense_peaks"] = MappingProxyType(dict(row["dense_peaks"]))
    row["measured"] = MappingProxyType(dict(measured_peaks(peaks_file)))
    return GpuFacts(**row)
