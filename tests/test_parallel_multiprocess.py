"""Sequence-parallel attention (Ulysses and gathered keys), GPipe and DiLoCo on 2 CPU ranks."""
import json
import os
import subprocess
import sys

import pytest

from dew_b200.parallel.pp import stage_slices
from dew_b200.parallel.sp import all_to_all_moves_less, stripe, unstripe

import torch

WORKER = os.path.join(os.path.dirname(__file__), "workers", "par_worker.py")


def test_two_rank_strategies():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29651", WORKER]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
    r = json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    for key in ("ulysses_out", "ulysses_dq", "ulysses_dk", "gathered_out", "pp_grad", "pp_loss", "diloco_spread"):
        assert r[key] < 1e-4, (key, r)
    assert r["diloco_took"] == 1.0


def test_helpers():
    assert [list(s) for s in stage_slices(7, 3)] == [[0, 1, 2], [3, 4], [5, 6]]
    x = torch.arange(16.0)[None, :, None]
    assert torch.equal(unstripe(stripe(x, 2), 2), x)
    assert stripe(x, 2)[0, :, 0].tolist()[:8] == [0, 1, 2, 3, 12, 13, 14, 15]
    assert all_to_all_moves_less(8192, 32, 8, 128, 8) and not all_to_all_moves_less(8192, 64, 1, 128, 2)


def test_link_probe_two_cpu_ranks():
    import json
    import os
    import subprocess
    import sys
    worker = os.path.join(os.path.dirname(__file__), "workers", "probe_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29671", worker]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
    r = json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    assert r["rows"] == 10 and r["positive"] and r["mem"] == 0 and r["table_lines"] == 11 and r["spread"] is False
    assert r["names"] == ["all_gather", "all_reduce", "all_to_all", "exchange", "reduce_scatter"]


def test_sequence_parallel_conv_band_scan_and_parallel_reductions():
    import json
    import os
    import subprocess
    import sys
    worker = os.path.join(os.path.dirname(__file__), "workers", "sp_ops_worker.py")
    for world, port in ((2, 29681), (3, 29682)):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
               "--master-port", str(port), worker]
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="1"))
        assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
        r = json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
        assert all(v < 1e-4 for v in r.values()), r
        assert {"conv_out", "band_out", "scan_out", "scan_state", "vce_loss", "norm"} <= set(r)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_sequence_parallel_exchanges_over_peer_memory():
    """The same worker on GPUs with a ``PeerLink``: halos, state hand-overs (forward and backward) and the row-statistic
    reductions each run as one kernel over NVLink peer memory, against the unsplit computation."""
    import json
    import os
    import subprocess
    import sys
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    worker = os.path.join(os.path.dirname(__file__), "workers", "sp_ops_worker.py")
    for world, port in ((2, 29691), (4, 29692)):
        if torch.cuda.device_count() < world:
            continue
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
               "--master-port", str(port), worker, "nccl"]
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="1"))
        assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
        r = json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
        assert -r.pop("launches") > 0, "no library kernel ran"
        assert all(v < 2e-3 for v in r.values()), r
        assert {"conv_out", "band_out", "scan_out", "scan_state", "vce_loss", "norm"} <= set(r)
