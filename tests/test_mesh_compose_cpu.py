"""``Trainer(mesh=MeshSpec(...))`` composes the parallel axes by itself: each composition, run on CPU ranks (gloo), takes the
same steps as one rank on the same global batch (reference behaviour: src/dew/distributed/placement.py:142-254, FSDP4xTP2 of
docs/performance.md:153-158, stage-local optimizer state of src/dew/training/stages.py)."""
import json
import os
import subprocess
import sys

import pytest

WORKER = os.path.join(os.path.dirname(__file__), "workers", "mesh_worker.py")


def _run(world, spec, optimizer="adamw", moe=False, clip="none", port=29700):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), WORKER, json.dumps(spec), optimizer, "moe" if moe else "dense", clip]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    line = next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))
    return json.loads(line[len("RESULT "):])


def _close(a, b, tol=2e-3):
    assert len(a["losses"]) == len(b["losses"])
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < tol * max(1.0, abs(x)), (a, b)


@pytest.fixture(scope="module")
def one_rank():
    return _run(1, {}, port=29700)


def test_fsdp_times_tensor_parallel(one_rank):
    got = _run(4, {"fsdp": 2, "tensor": 2}, port=29701)
    assert got["engine"] == "FSDPEngine"
    _close(one_rank, got)


def test_tensor_parallel_alone_with_clipping():
    ref = _run(1, {}, clip="0.5", port=29702)
    got = _run(2, {"tensor": 2}, clip="0.5", port=29703)
    _close(ref, got)


def test_hybrid_sharding_replicas(one_rank):
    got = _run(4, {"fsdp": 2, "replicas": 2}, port=29704)
    assert got["engine"] == "FSDPEngine"
    _close(one_rank, got)


def test_pipeline_stages_with_stage_local_state(one_rank):
    got = _run(2, {"stage": 2}, port=29705)
    assert got["engine"] == "PipelineEngine"
    _close(one_rank, got)


def test_pipeline_times_data_parallel(one_rank):
    got = _run(4, {"stage": 2}, port=29706)            # the two ranks the stages leave become the data axis
    _close(one_rank, got)


def test_data_parallel_with_an_optimizer_the_sharded_kernel_lacks():
    ref = _run(1, {}, optimizer="lion", port=29707)
    got = _run(2, {"fsdp": 2}, optimizer="lion", port=29708)
    assert got["engine"] == "DataParallelEngine"
    _close(ref, got)


def test_expert_parallel_inside_fsdp():
    ref = _run(1, {}, moe=True, port=29709)
    got = _run(4, {"expert": 2, "fsdp": 2}, moe=True, port=29710)
    assert got["engine"] == "FSDPEngine"
    _close(ref, got, tol=5e-3)


def test_local_checkpoint_lost_by_one_rank_is_recovered_from_its_replica(tmp_path):
    """Hybrid sharding keeps every shard on two ranks: a rank that lost its local (emergency) checkpoint gets its shards from
    the other holder; when both holders lost theirs the step is refused (src/dew/checkpoints/_replicas.py)."""
    worker = os.path.join(os.path.dirname(__file__), "workers", "replica_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
           "--master-port", "29720", worker, str(tmp_path)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    r = json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    assert r["recovered"] and r["refused"] and len(r["holders_of_1"]) == 2 and r["steps_rank0"] == [2], r
