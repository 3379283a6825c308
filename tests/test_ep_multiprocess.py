"""Expert parallelism over 2 and 4 CPU ranks equals the unsharded mixture-of-experts layer."""
import json
import os
import subprocess
import sys

import pytest

WORKER = os.path.join(os.path.dirname(__file__), "workers", "ep_worker.py")


@pytest.mark.parametrize("world,port", [(2, 29641), (4, 29642)])
def test_expert_parallel_matches_single_process(world, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), WORKER]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
    r = json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    assert r["out_err"] < 1e-5 and r["dx_err"] < 1e-4 and r["dw_err"] < 1e-4, r


def test_expert_parallel_with_gathered_weights_matches_single_process():
    """``dispatch='global'``: the experts' weights are all-gathered and every rank runs its own tokens; the weight gradients
    return to their owners by a reduce-scatter."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29655", WORKER, "global"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
    r = json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    assert r["out_err"] < 1e-5 and r["dx_err"] < 1e-4 and r["dw_err"] < 1e-4, r


def _run_moe(world, port):
    worker = os.path.join(os.path.dirname(__file__), "workers", "moe_fsdp_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), worker]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
    return json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])


def test_moe_lm_trains_under_fsdp_with_expert_parallel_units():
    """Experts split over 2 ranks as rank-local units of the FSDP engine (no reduction, local AdamW), the rest sharded:
    the same losses and final weights as one process holding every expert."""
    one, two = _run_moe(1, 29651), _run_moe(2, 29652)
    assert two["local_units"] == 2 and two["losses"][-1] < two["losses"][0]
    for a, b in zip(one["losses"], two["losses"]):
        assert abs(a - b) < 2e-3 * max(1.0, abs(a)), (one, two)
    assert abs(one["digest"] - two["digest"]) < 1e-3 * one["digest"], (one["digest"], two["digest"])
    assert two["experts"] == one["experts"]              # the export concatenates every rank's experts


@pytest.mark.gpu
@pytest.mark.multigpu
def test_expert_parallel_two_gpus_peer_memory_exchange():
    """Dispatch by peer stores into the owners' expert-sorted buffers and combine by peer loads (one kernel each), against
    the NCCL all-to-all form of the same layer; three calls in a row so that buffers and flags are reused."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    worker = os.path.join(os.path.dirname(__file__), "workers", "ep_gpu_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29661", worker]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="2"))
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    r = json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    assert max(r["errs"]) < 5e-2, r
