"""Tensor parallelism: sharded model == full model, on 2 CPU ranks (gloo) and, with GPUs, through the fused peer-memory
all-reduce + residual + RMSNorm kernel."""
import json
import os
import subprocess
import sys

import pytest
import torch

WORKER = os.path.join(os.path.dirname(__file__), "workers", "tp_worker.py")


def _run(world, backend, port, mode="auto"):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), WORKER, backend]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="2", DEWB_TP_ALLREDUCE=mode))
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    return json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])


def test_tensor_parallel_two_cpu_ranks():
    r = _run(2, "gloo", 29631)
    assert r["err"] < 1e-5 and r["same_tokens"]


@pytest.mark.gpu
@pytest.mark.multigpu
def test_tensor_parallel_two_gpus_fused_allreduce():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    for i, mode in enumerate(("auto", "twoshot", "oneshot")):        # low-latency lines, two flagged shots, one-shot pull
        r = _run(2, "nccl", 29632 + 20 * i, mode)
        assert r["err"] < 3e-2, (mode, r)
        assert r["allreduce_worst"] < 1.2e-2, (mode, r)          # bf16 rounding of the sum and of the normalised row


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("world", [4, 8])
def test_tensor_parallel_more_gpus_fused_allreduce(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    for i, mode in enumerate(("auto", "twoshot")):
        r = _run(world, "nccl", 29632 + world + 20 * i, mode)
        assert r["err"] < 3e-2 and r["allreduce_worst"] < 1.2e-2, (mode, r)


def _run_spl(world, backend, port, *extra):
    worker = os.path.join(os.path.dirname(__file__), "workers", "spl_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), worker, backend, *[str(e) for e in extra]]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="2"))
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    return json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])


def test_sequence_parallel_linear_two_cpu_ranks():
    """all-gather -> matmul and matmul -> reduce-scatter (+ residual), host-side path, against the unsharded products."""
    r = _run_spl(2, "gloo", 29641)
    assert max(r["errs"]) < 1e-5, r


@pytest.mark.gpu
@pytest.mark.multigpu
def test_sequence_parallel_linear_two_gpus_fused_kernels():
    """The same products as ONE kernel each over peer memory (TMA reads of the peer's shard; epilogue stores into the
    owner's partial buffer), three calls in a row so that the buffers are reused."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    r = _run_spl(2, "nccl", 29642, 512, 256, 384)
    assert max(r["errs"]) < 2e-2, r
    r = _run_spl(2, "nccl", 29643, 1024, 512, 1024)
    assert max(r["errs"]) < 2e-2, r
