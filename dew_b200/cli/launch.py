"""``dewb launch -- cmd``: spawn one process per GPU on this host (and, with ``--hosts``, over ssh on others), prefix
their output with the rank, and end the whole pool when one process dies.

Parity: src/dew/_cli/launch.py (``Launch`` :102, ``gpu_count`` :442, ``supervise`` :562-666; behaviour
docs/guides/multi-node.md:52-84: 10 s grace when a rank dies, 300 s after a signal so ranks can checkpoint, rank 0
ends last).
"""
from __future__ import annotations

import argparse
import os
import shlex
import signal
import subprocess
import sys
import threading
import time
from typing import Dict, List, Optional, Sequence

DEATH_GRACE = 10.0
SIGNAL_GRACE = 300.0


def gpu_count() -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis is not None:
        return len([v for v in vis.split(",") if v.strip()])
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=10).stdout
        return max(1, len([l for l in out.splitlines() if l.startswith("GPU ")]))
    except Exception:
        return 1


def plan(command: Sequence[str], processes_per_host: int, hosts: Sequence[str], port: int, extra_env: Dict[str, str]) -> List[dict]:
    """One entry per process: its rank, host, environment and command line."""
    hosts = list(hosts) or ["127.0.0.1"]
    world = processes_per_host * len(hosts)
    out = []
    for h, host in enumerate(hosts):
        for l in range(processes_per_host):
            rank = h * processes_per_host + l
            env = {"RANK": str(rank), "LOCAL_RANK": str(l), "WORLD_SIZE": str(world), "LOCAL_WORLD_SIZE": str(processes_per_host),
                   "MASTER_ADDR": hosts[0], "MASTER_PORT": str(port), **extra_env}
            out.append({"rank": rank, "host": host, "env": env, "command": list(command)})
    return out


def _pump(stream, rank: int, sink) -> None:
    for line in iter(stream.readline, ""):
        sink.write(f"[{rank}] {line}")
        sink.flush()


def supervise(procs: List[subprocess.Popen], death_grace: float = DEATH_GRACE, signal_grace: float = SIGNAL_GRACE) -> int:
    """Wait for the pool; when one process exits non-zero give the rest ``death_grace`` seconds, then kill them (rank 0
    last). SIGINT / SIGTERM are forwarded and the pool gets ``signal_grace`` seconds to checkpoint."""
    signalled = {"at": None}

    def forward(signum, frame):
        signalled["at"] = time.monotonic()
        for p in procs:
            if p.poll() is None:
                p.send_signal(signum)
    for s in (signal.SIGINT, signal.SIGTERM):
        try:
            signal.signal(s, forward)
        except ValueError:
            pass
    first_bad: Optional[int] = None
    died_at: Optional[float] = None
    while True:
        codes = [p.poll() for p in procs]
        if all(c is not None for c in codes):
            break
        bad = next((c for c in codes if c not in (None, 0)), None)
        if bad is not None and first_bad is None:
            first_bad, died_at = bad, time.monotonic()
        now = time.monotonic()
        expired = (died_at is not None and now - died_at > death_grace) or \
                  (signalled["at"] is not None and now - signalled["at"] > signal_grace)
        if expired:
            for p in reversed(procs):                      # rank 0 last
                if p.poll() is None:
                    p.kill()
        time.sleep(0.05)
    codes = [p.returncode for p in procs]
    if first_bad is not None:
        return first_bad
    return next((c for c in codes if c != 0), 0)


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="dewb launch")
    ap.add_argument("--hosts", default="", help="comma-separated hosts (ssh); default this host only")
    ap.add_argument("--processes-per-host", type=int, default=None)
    ap.add_argument("--port", type=int, default=29400)
    ap.add_argument("--env", action="append", default=[], help="K=V passed to every process")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("command", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    cmd = [c for c in args.command if c != "--"] if args.command and args.command[0] == "--" else list(args.command)
    if not cmd:
        ap.error("give the command after --")
    hosts = [h for h in args.hosts.split(",") if h]
    per = args.processes_per_host or gpu_count()
    extra = dict(kv.split("=", 1) for kv in args.env)
    entries = plan(cmd, per, hosts, args.port, extra)
    if args.dry_run:
        for e in entries:
            print(f"rank {e['rank']} on {e['host']}: " + " ".join(f"{k}={v}" for k, v in e["env"].items()) + " " + " ".join(map(shlex.quote, e["command"])))
        return 0
    procs, threads = [], []
    for e in entries:
        if e["host"] in ("127.0.0.1", "localhost") or not hosts:
            p = subprocess.Popen(e["command"], env={**os.environ, **e["env"]}, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        else:
            remote = " ".join(f"{k}={shlex.quote(v)}" for k, v in e["env"].items()) + " " + " ".join(map(shlex.quote, e["command"]))
            p = subprocess.Popen(["ssh", e["host"], f"cd {shlex.quote(os.getcwd())} && {remote}"], stdout=subprocess.PIPE,
                                 stderr=subprocess.STDOUT, text=True)
        t = threading.Thread(target=_pump, args=(p.stdout, e["rank"], sys.stdout), daemon=True)
        t.start()
        procs.append(p); threads.append(t)
    code = supervise(procs)
    for t in threads:
        t.join(timeout=1.0)
    return code


if __name__ == "__main__":
    sys.exit(main())
