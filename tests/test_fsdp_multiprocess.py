"""FSDP engine across processes: 2 CPU ranks (gloo) must take the same steps as 1 rank on the same global batch; on a
box with >= 2 GPUs the fused peer-memory kernel must match too."""
import json
import os
import subprocess
import sys

import pytest
import torch

WORKER = os.path.join(os.path.dirname(__file__), "workers", "fsdp_worker.py")


def _run(world, backend, clip="none", port=29611, mode="resident"):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), WORKER, backend, clip, mode]
    env = dict(os.environ, OMP_NUM_THREADS="2")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    line = next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))
    return json.loads(line[len("RESULT "):])


def test_fsdp_two_cpu_ranks_match_one_rank():
    one = _run(1, "gloo", port=29611)
    two = _run(2, "gloo", port=29612)
    # the same global batch, split over ranks: pooled losses and the updated weights agree
    assert two["losses"][-1] < two["losses"][0]
    for a, b in zip(one["losses"], two["losses"]):
        assert abs(a - b) < 2e-3 * max(1.0, abs(a)), (one, two)
    assert abs(one["digest"] - two["digest"]) < 1e-3 * one["digest"]
    assert one["arena_ok"] and two["arena_ok"]


def test_fully_sharded_engine_matches_one_rank_on_cpu_ranks():
    """Parameters and gradients as shards, gathered and reduced unit by unit, every microbatch: the same steps as one rank."""
    one = _run(1, "gloo", port=29614)
    two = _run(2, "gloo", port=29615, mode="sharded")
    for a, b in zip(one["losses"], two["losses"]):
        assert abs(a - b) < 2e-3 * max(1.0, abs(a)), (one, two)
    assert abs(one["digest"] - two["digest"]) < 1e-3 * one["digest"]
    clipped_ref = _run(2, "gloo", clip="0.5", port=29616)
    clipped = _run(2, "gloo", clip="0.5", port=29617, mode="sharded")
    for a, b in zip(clipped_ref["losses"], clipped["losses"]):
        assert abs(a - b) < 2e-3 * max(1.0, abs(a)), (clipped_ref, clipped)


def test_fsdp_two_cpu_ranks_with_clipping():
    two = _run(2, "gloo", clip="0.5", port=29613)
    assert two["losses"][-1] < two["losses"][0]


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_fsdp_gpus_fused_kernel(world):
    """The fused reduce-scatter + AdamW + all-gather kernel on `world` GPUs against one GPU on the same global batch, and
    the compute copy read straight after a step against the gathered masters."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    one = _run(1, "nccl", port=29621)
    many = _run(world, "nccl", port=29622 + world)
    assert many["losses"][-1] < many["losses"][0] and many["arena_ok"]
    for a, b in zip(one["losses"], many["losses"]):
        assert abs(a - b) < 3e-2 * max(1.0, abs(a)), (one, many)
    assert abs(one["digest"] - many["digest"]) < 5e-3 * one["digest"]
    clipped = _run(world, "nccl", clip="0.5", port=29640 + world)
    assert clipped["losses"][-1] < clipped["losses"][0]
    # the fully sharded engine (gathers and reductions per unit per microbatch over peer memory) takes the same steps
    sharded = _run(world, "nccl", port=29660 + world, mode="sharded")
    for a, b in zip(many["losses"], sharded["losses"]):
        assert abs(a - b) < 3e-2 * max(1.0, abs(a)), (many, sharded)
    assert abs(many["digest"] - sharded["digest"]) < 5e-3 * many["digest"]


def _run_ckpt(world, directory, steps, port):
    worker = os.path.join(os.path.dirname(__file__), "workers", "ckpt_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), worker, str(directory), str(steps)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="2"))
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    line = next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))
    return json.loads(line[len("RESULT "):])


def test_fsdp_checkpoint_resumes_at_another_world_size(tmp_path):
    """5 uninterrupted steps on 2 ranks == 3 steps on 2 ranks, checkpoint, then 2 more steps on ONE rank: the checkpoint
    holds whole trees, so it restores into any sharding (weights, Adam moments, EMA, data position)."""
    straight = _run_ckpt(2, tmp_path / "a", 5, 29631)
    first = _run_ckpt(2, tmp_path / "b", 3, 29632)
    assert first["step"] == 3
    resumed = _run_ckpt(1, tmp_path / "b", 5, 29633)
    assert resumed["step"] == 5 and len(resumed["losses"]) == 2
    assert abs(resumed["digest"] - straight["digest"]) < 2e-4 * straight["digest"], (resumed, straight)
    assert abs(resumed["ema"] - straight["ema"]) < 2e-4 * straight["ema"]
    for a, b in zip(straight["losses"][3:], resumed["losses"]):
        assert abs(a - b) < 2e-3 * max(1.0, abs(a))
