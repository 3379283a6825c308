"""Agreements, failure publication and the launcher, all on the host (no GPU)."""
import os
import subprocess
import sys
import threading
import time

import pytest

from dew_b200.cli import launch
from dew_b200.parallel.clusters import OpenMPI, Slurm, TorchRun, detected_environment
from dew_b200.parallel.coordination import AgreementTimeout, DictStore, PeerFailure, Pool


def _pools(n, patience=5.0):
    store = DictStore()
    return [Pool(store, r, n, patience=patience) for r in range(n)]


def _run_all(pools, fn):
    out, errs = [None] * len(pools), [None] * len(pools)

    def work(i):
        try:
            out[i] = fn(pools[i])
        except BaseException as e:
            errs[i] = e
    ts = [threading.Thread(target=work, args=(i,)) for i in range(len(pools))]
    [t.start() for t in ts]
    [t.join() for t in ts]
    return out, errs


def test_gather_agreed_and_agreed_same():
    pools = _pools(3)
    out, errs = _run_all(pools, lambda p: p.gather("x", p.rank * 10))
    assert errs == [None] * 3 and out == [[0, 10, 20]] * 3
    out, _ = _run_all(pools, lambda p: p.agreed_next("step", 100 + p.rank))
    assert out == [102] * 3
    out, _ = _run_all(pools, lambda p: p.agreed("decide", lambda: "from rank 0"))
    assert out == ["from rank 0"] * 3
    _, errs = _run_all(pools, lambda p: p.agreed_same("cfg", {"lr": 1e-3 if p.rank != 2 else 2e-3}))
    assert all(isinstance(e, RuntimeError) and "[2]" in str(e) for e in errs)


def test_a_failed_rank_releases_its_waiting_peers():
    pools = _pools(3, patience=30.0)

    def fn(p):
        if p.rank == 1:
            time.sleep(0.1)
            p.publish_failure(ValueError("loader raised"))
            return "failed"
        return p.gather("phase", 1)           # would wait for rank 1 forever
    t0 = time.monotonic()
    out, errs = _run_all(pools, fn)
    assert time.monotonic() - t0 < 5.0
    assert isinstance(errs[0], PeerFailure) and errs[0].rank == 1 and "loader raised" in str(errs[0])
    assert isinstance(errs[2], PeerFailure)


def test_a_rank_that_never_joins_times_out():
    pools = _pools(2, patience=0.3)
    with pytest.raises(AgreementTimeout):
        pools[0].gather("lonely", 1)


def test_cluster_detection():
    assert isinstance(detected_environment({"RANK": "1", "WORLD_SIZE": "4", "MASTER_ADDR": "10.0.0.1", "MASTER_PORT": "1234", "LOCAL_RANK": "1"}), TorchRun)
    j = OpenMPI({"OMPI_COMM_WORLD_SIZE": "8", "OMPI_COMM_WORLD_RANK": "3", "OMPI_COMM_WORLD_LOCAL_RANK": "3"}).joining()
    assert (j.count, j.rank, j.local_rank) == (8, 3, 3)
    j = Slurm({"SLURM_PROCID": "5", "SLURM_NTASKS": "16", "SLURM_LOCALID": "1", "SLURM_JOB_NODELIST": "gpu[07-09,12]", "SLURM_JOB_ID": "42"}).joining()
    assert j.coordinator.startswith("gpu07:") and j.rank == 5
    assert detected_environment({}) is None


def test_launcher_plan_and_pool_teardown(tmp_path):
    entries = launch.plan(["python", "train.py"], 2, ["a", "b"], 29400, {"X": "1"})
    assert [e["rank"] for e in entries] == [0, 1, 2, 3] and entries[3]["env"]["LOCAL_RANK"] == "1" and entries[2]["host"] == "b"
    # rank 1 dies; rank 0 would sleep for a minute: the supervisor must end it within the grace period
    script = tmp_path / "w.py"
    script.write_text("import os, sys, time\nif os.environ['RANK'] == '1':\n    sys.exit(3)\ntime.sleep(60)\n")
    procs = [subprocess.Popen([sys.executable, str(script)], env={**os.environ, "RANK": str(r)}) for r in range(2)]
    t0 = time.monotonic()
    code = launch.supervise(procs, death_grace=0.5)
    assert code == 3 and time.monotonic() - t0 < 10
