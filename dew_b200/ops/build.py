"""Builds the CUDA library in-tree: every ``csrc/kernels/*.cu`` -> object -> ``dew_b200/ops/libdewb.so``.

The kernels are plain CUDA with ``extern "C"`` launchers (no torch headers), so a file compiles in seconds;
``nvcc`` cross-compiles for ``sm_100a`` on a machine without a GPU.  Python reaches the launchers through
``ctypes`` (``dew_b200.ops.library``).  Run ``python -m dew_b200.ops.build`` or call :func:`build`.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List

ROOT = Path(__file__).resolve().parents[2]
CSRC = ROOT / "csrc"
OUT_DIR = Path(__file__).resolve().parent
OBJ_DIR = OUT_DIR / "_obj"
LIB = OUT_DIR / "libdewb.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
              "--expt-relaxed-constexpr"]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def sources() -> List[Path]:
    return sorted((CSRC / "kernels").glob("*.cu"))


def _digest(path: Path) -> str:
    h = hashlib.sha256()
    h.update(path.read_bytes())
    for folder in ("common", "include"):                       # every header a kernel file may include
        for hdr in sorted((CSRC / folder).glob("*")):
            h.update(hdr.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _compile(src: Path, verbose: bool) -> Path:
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    obj = OBJ_DIR / f"{src.stem}.{_digest(src)}.o"
    if obj.exists():
        return obj
    for stale in OBJ_DIR.glob(f"{src.stem}.*.o"):
        stale.unlink()
    cmd = [nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = OBJ_DIR / f"{src.stem}.ptxas.log"
    log.write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(f"[dew_b200.build] compiled {src.name}", file=sys.stderr)
    return obj


def build(verbose: bool = True, force: bool = False) -> Path:
    """Compile what changed and link; returns the library path."""
    if force and OBJ_DIR.exists():
        shutil.rmtree(OBJ_DIR)
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(srcs)))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), srcs))
    stamp = OBJ_DIR / "link.stamp"
    want = " ".join(o.name for o in objs)
    if LIB.exists() and stamp.exists() and stamp.read_text() == want:
        return LIB
    cmd = [nvcc(), "-shared", *ARCH_FLAGS, "-Xcompiler", "-fPIC", "-o", str(LIB), *map(str, objs), "-cudart", "static"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    stamp.write_text(want)
    if verbose:
        print(f"[dew_b200.build] linked {LIB}", file=sys.stderr)
    return LIB


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel, from the last compile of each file."""
    out = []
    for log in sorted(OBJ_DIR.glob("*.ptxas.log")):
        out.append(f"== {log.stem}\n{log.read_text()}")
    return "\n".join(out)


def kernel_resources() -> dict:
    """``{(file, kernel symbol): {"registers", "spill_stores", "spill_loads", "stack"}}`` parsed from the ptxas logs of the
    last compile (the resource gate of the tests reads this: a kernel that starts to spill shows up here, before any GPU run)."""
    import re
    found = {}
    for log in sorted(OBJ_DIR.glob("*.ptxas.log")):
        entry = None
        for line in log.read_text().splitlines():
            m = re.search(r"Compiling entry function '([^']+)' for 'sm_100a'", line)
            if m:
                entry = (log.name.split(".")[0], m.group(1))
                found[entry] = {"registers": 0, "spill_stores": 0, "spill_loads": 0, "stack": 0}
                continue
            if entry is None:
                continue
            m = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", line)
            if m:
                found[entry].update(stack=int(m.group(1)), spill_stores=int(m.group(2)), spill_loads=int(m.group(3)))
            m = re.search(r"Used (\d+) registers", line)
            if m:
                found[entry]["registers"] = int(m.group(1))
    return found


if __name__ == "__main__":
    build(verbose=True, force="--force" in sys.argv)
    if "--report" in sys.argv:
        print(ptxas_report())
