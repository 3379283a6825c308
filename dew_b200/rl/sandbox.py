"""Run untrusted programs and tool sessions in bounded Linux subprocesses.

A ``Program`` holds the files to write into a fresh temporary directory, an argv to run there without a shell, and the text for
its stdin.  A runner executes one program under ``SandboxLimits`` (RLIMIT_CPU, RLIMIT_AS, a wall-clock deadline, capped output)
and reports an ``Outcome``: how it ended (``Verdict``), its exit code, its capped output and the seconds it took.
``SandboxFleet`` runs programs on several worker threads at once, each program in its own process group which is killed whole
when the program ends, however it ends; a verifiable reward uses it to score completions (``outputs_match``, ``MathReward``).
``SubprocessEnvironment`` is an episode environment whose worker is a JSON-lines process the caller chooses.

The workers run under the caller's OS permissions: CPU, memory, time and output are bounded, the filesystem and the network are
not isolated, so hostile code needs an outer boundary (a container: ``ContainerRunner``).  Nothing selects or runs a sandbox by
default.

Reference: src/dew/rl/sandbox.py (``SandboxLimits``, ``SubprocessEnvironment``, ``Verdict``, ``Program``, ``Outcome``,
``ProcessRunner``, ``ContainerRunner``, ``SandboxFleet``, ``outputs_match``, ``MathReward``).
"""
from __future__ import annotations

import enum
import json
import os
import re
import shutil
import signal
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from fractions import Fraction
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

_LAUNCHER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_sandbox_exec.py")


@dataclass(frozen=True)
class SandboxLimits:
    cpu_seconds: int = 10
    memory_bytes: int = 1 << 30
    wall_seconds: float = 20.0
    output_bytes: int = 1 << 20
    file_bytes: int = 64 << 20
    message_bytes: int = 1 << 20


class Verdict(enum.Enum):
    COMPLETED = "completed"          # exited by itself (any exit code)
    TIMED_OUT = "timed_out"          # the wall deadline or the CPU limit
    OUTPUT_EXCEEDED = "output_exceeded"
    KILLED = "killed"                # ended by a signal (memory limit included)


@dataclass(frozen=True)
class Program:
    files: Mapping[str, str]
    command: Tuple[str, ...]
    stdin: str = ""

    def __post_init__(self):
        if not self.command or not all(isinstance(a, str) for a in self.command):
            raise ValueError("a program's command is a nonempty argv of strings")
        for name in self.files:
            norm = os.path.normpath(name)
            if os.path.isabs(name) or norm.startswith("..") or norm in (".", ""):
                raise ValueError(f"a program's files are relative paths inside its directory, got {name!r}")


@dataclass(frozen=True)
class Outcome:
    verdict: Verdict
    exit_code: Optional[int]
    stdout: str
    stderr: str
    seconds: float

    @property
    def ok(self) -> bool:
        return self.verdict is Verdict.COMPLETED and self.exit_code == 0


def _kill_group(proc: subprocess.Popen) -> None:
    try:
        os.killpg(proc.pid, signal.SIGKILL)          # the process started its own session: pid == pgid
    except (ProcessLookupError, PermissionError):
        pass


def launched(command: Sequence[str], directory: str, limits: SandboxLimits, env: Optional[Mapping[str, str]] = None) -> subprocess.Popen:
    argv = [sys.executable, "-I", _LAUNCHER, str(limits.cpu_seconds), str(limits.memory_bytes), str(limits.file_bytes), *command]
    clean = {"PATH": os.environ.get("PATH", "/usr/bin:/bin"), "HOME": directory, "LANG": "C.UTF-8", **(dict(env) if env else {})}
    return subprocess.Popen(argv, cwd=directory, env=clean, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                            start_new_session=True)


class Runner:
    python: Tuple[str, ...] = (sys.executable, "-I")

    def run(self, program: Program, limits: SandboxLimits) -> Outcome:
        raise NotImplementedError


def _write_files(directory: str, files: Mapping[str, str]) -> None:
    for name, text in files.items():
        path = os.path.join(directory, name)
        os.makedirs(os.path.dirname(path) or directory, exist_ok=True)
        with open(path, "w") as f:
            f.write(text)


def _pump(stream, cap: int, sink: List[bytes], over: threading.Event) -> None:
    held = 0
    while True:
        chunk = stream.read(65536)
        if not chunk:
            return
        if held < cap:
            sink.append(chunk[: cap - held])
        held += len(chunk)
        if held > cap:
            over.set()


class ProcessRunner(Runner):
    """Each program as a resource-limited process in a temporary directory.  The whole process group is killed at the wall
    deadline, on excess output and after a normal exit, so no child the program forked outlives it."""

    def run(self, program: Program, limits: SandboxLimits) -> Outcome:
        directory = tempfile.mkdtemp(prefix="sandbox-")
        began = time.monotonic()
        try:
            _write_files(directory, program.files)
            proc = launched(program.command, directory, limits)
            out: List[bytes] = []
            err: List[bytes] = []
            over = threading.Event()
            pumps = [threading.Thread(target=_pump, args=(proc.stdout, limits.output_bytes, out, over), daemon=True),
                     threading.Thread(target=_pump, args=(proc.stderr, limits.output_bytes, err, over), daemon=True)]
            for p in pumps:
                p.start()
            try:
                proc.stdin.write(program.stdin.encode())
                proc.stdin.close()
            except (BrokenPipeError, OSError):
                pass
            verdict = None
            deadline = began + limits.wall_seconds
            while proc.poll() is None:
                if over.is_set():
                    verdict = Verdict.OUTPUT_EXCEEDED
                    break
                if time.monotonic() > deadline:
                    verdict = Verdict.TIMED_OUT
                    break
                time.sleep(0.005)
            _kill_group(proc)
            proc.wait()
            for p in pumps:
                p.join(timeout=1.0)
            code = proc.returncode
            if verdict is None:
                if over.is_set():
                    verdict = Verdict.OUTPUT_EXCEEDED
                elif code is not None and code < 0:
                    verdict = Verdict.TIMED_OUT if -code == signal.SIGXCPU else Verdict.KILLED
                else:
                    verdict = Verdict.COMPLETED
            return Outcome(verdict, code if verdict is Verdict.COMPLETED else None, b"".join(out).decode("utf-8", "replace"),
                           b"".join(err).decode("utf-8", "replace"), time.monotonic() - began)
        finally:
            shutil.rmtree(directory, ignore_errors=True)


class ContainerRunner(Runner):
    """Each program in a fresh container of ``image`` with no network; the job directory is mounted read-only at ``/work``.
    ``runtime`` is a Docker-compatible CLI; it is looked up when a program runs, not when the runner is built."""
    python = ("python3", "-I")

    def __init__(self, image: str, runtime: str = "docker"):
        self.image, self.runtime = image, runtime

    def argv(self, directory: str, program: Program, limits: SandboxLimits) -> List[str]:
        return [self.runtime, "run", "--rm", "-i", "--network", "none", "--read-only", "--tmpfs", "/tmp:size=64m",
                "--memory", str(limits.memory_bytes), "--pids-limit", "128", "--cpus", "1", "-v", f"{directory}:/work:ro", "-w", "/work",
                self.image, *program.command]

    def run(self, program: Program, limits: SandboxLimits) -> Outcome:
        if shutil.which(self.runtime) is None:
            raise RuntimeError(f"container runtime {self.runtime!r} is not installed")
        directory = tempfile.mkdtemp(prefix="sandbox-")
        began = time.monotonic()
        try:
            _write_files(directory, program.files)
            try:
                done = subprocess.run(self.argv(directory, program, limits), input=program.stdin.encode(), capture_output=True,
                                      timeout=limits.wall_seconds)
            except subprocess.TimeoutExpired as e:
                return Outcome(Verdict.TIMED_OUT, None, (e.stdout or b"").decode("utf-8", "replace")[: limits.output_bytes], "", time.monotonic() - began)
            return Outcome(Verdict.COMPLETED, done.returncode, done.stdout.decode("utf-8", "replace")[: limits.output_bytes],
                           done.stderr.decode("utf-8", "replace")[: limits.output_bytes], time.monotonic() - began)
        finally:
            shutil.rmtree(directory, ignore_errors=True)


def usable_cpus() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


class SandboxFleet:
    def __init__(self, runner: Optional[Runner] = None, workers: Optional[int] = None, limits: SandboxLimits = SandboxLimits()):
        self.runner = runner or ProcessRunner()
        self.workers = workers or usable_cpus()
        self.limits = limits
        self._pool = ThreadPoolExecutor(self.workers, thread_name_prefix="sandbox")

    def run(self, programs: Sequence[Program]) -> List[Outcome]:
        return list(self._pool.map(lambda p: self.runner.run(p, self.limits), programs))

    def python(self, source: str, stdin: str = "") -> Program:
        return Program({"main.py": source}, (*self.runner.python, "main.py"), stdin)

    def close(self) -> None:
        self._pool.shutdown(wait=True)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def outputs_match(outcome: Outcome, expected: str) -> bool:
    """Whether the program completed with exit code 0 and its stdout equals ``expected``, ignoring whitespace around the whole
    output and at the end of each line."""
    if not outcome.ok:
        return False
    norm = lambda s: [line.rstrip() for line in s.strip().splitlines()]
    return norm(outcome.stdout) == norm(expected)


# ------------------------------------------------------------------------------------------------ verifiable rewards
_NUMBER = re.compile(r"-?\d+(?:,\d{3})*(?:\.\d+)?(?:/\d+)?")


def _boxed(text: str) -> Optional[str]:
    at = text.rfind("\\boxed{")
    if at < 0:
        return None
    depth, start = 0, at + len("\\boxed{")
    for i in range(start, len(text)):
        if text[i] == "{":
            depth += 1
        elif text[i] == "}":
            if depth == 0:
                return text[start:i]
            depth -= 1
    return None


def _rational(text: str) -> Optional[Fraction]:
    t = text.strip().replace(",", "").replace("$", "").replace("\\!", "").strip()
    m = re.fullmatch(r"\\d?frac\{(-?\d+)\}\{(\d+)\}", t)
    if m:
        return Fraction(int(m.group(1)), int(m.group(2))) if int(m.group(2)) else None
    if t.endswith("%"):
        inner = _rational(t[:-1])
        return None if inner is None else inner / 100
    try:
        return Fraction(t)
    except (ValueError, ZeroDivisionError):
        return None


class MathReward:
    """1.0 when the final answer equals the reference as a rational number, else 0.0.  The answer is the last ``\\boxed{}`` of
    the completion; with ``require_boxed=False`` a completion without one uses its last number."""

    def __init__(self, require_boxed: bool = True):
        self.require_boxed = require_boxed

    def answer(self, completion: str) -> Optional[Fraction]:
        boxed = _boxed(completion)
        if boxed is not None:
            return _rational(boxed)
        if self.require_boxed:
            return None
        found = _NUMBER.findall(completion)
        return _rational(found[-1]) if found else None

    def __call__(self, completion: str, reference: str) -> float:
        got, want = self.answer(completion), _rational(str(reference))
        return float(got is not None and want is not None and got == want)


class ProgramReward:
    """Scores code completions by running them: the completion's last fenced code block is run against each ``(stdin, expected
    stdout)`` case on the fleet; the reward is the share of cases whose output matches."""

    def __init__(self, fleet: SandboxFleet):
        self.fleet = fleet

    @staticmethod
    def code_of(completion: str) -> Optional[str]:
        blocks = re.findall(r"```(?:python|py)?\n(.*?)```", completion, flags=re.S)
        return blocks[-1] if blocks else None

    def __call__(self, completions: Sequence[str], cases: Sequence[Sequence[Tuple[str, str]]]) -> List[float]:
        programs, owner = [], []
        for i, (c, tests) in enumerate(zip(completions, cases)):
            code = self.code_of(c)
            if code is None:
                continue
            for stdin, _ in tests:
                programs.append(self.fleet.python(code, stdin))
                owner.append(i)
        outcomes = self.fleet.run(programs)
        score = [0.0] * len(completions)
        at: Dict[int, int] = {}
        for i, o in zip(owner, outcomes):
            k = at.get(i, 0)
            at[i] = k + 1
            score[i] += float(outputs_match(o, cases[i][k][1])) / max(1, len(cases[i]))
        return score


# ------------------------------------------------------------------------------------------------ an environment in a worker process
class SubprocessEnvironment:
    """An episode environment run as a JSON-lines worker process: each request ``{"op": "reset" | "step", ...}`` is one line on
    the worker's stdin and each reply one line on its stdout, both capped at ``limits.message_bytes``.  The worker is killed
    with its process group on ``close`` and at the wall deadline of a reply."""

    def __init__(self, command: Sequence[str], limits: SandboxLimits = SandboxLimits(), files: Optional[Mapping[str, str]] = None):
        self.limits = limits
        self.directory = tempfile.mkdtemp(prefix="sandbox-env-")
        _write_files(self.directory, files or {})
        self.proc = launched(tuple(command), self.directory, limits)
        self._lock = threading.Lock()

    def _ask(self, request: Mapping[str, Any]) -> Dict[str, Any]:
        line = json.dumps(request)
        if len(line) > self.limits.message_bytes:
            raise ValueError("the request is past the message limit")
        with self._lock:
            if self.proc.poll() is not None:
                raise RuntimeError(f"the worker has exited with code {self.proc.returncode}")
            self.proc.stdin.write(line.encode() + b"\n")
            self.proc.stdin.flush()
            reply: List[bytes] = []
            reader = threading.Thread(target=lambda: reply.append(self.proc.stdout.readline(self.limits.message_bytes + 1)), daemon=True)
            reader.start()
            reader.join(self.limits.wall_seconds)
            if reader.is_alive() or not reply or not reply[0]:
                self.close()
                raise TimeoutError("the worker did not answer inside the wall deadline")
            if len(reply[0]) > self.limits.message_bytes:
                self.close()
                raise ValueError("the worker's reply is past the message limit")
            return json.loads(reply[0])

    def reset(self, **options) -> Dict[str, Any]:
        return self._ask({"op": "reset", **options})

    def step(self, action: Any) -> Dict[str, Any]:
        return self._ask({"op": "step", "action": action})

    def close(self) -> None:
        if self.proc.poll() is None:
            _kill_group(self.proc)
            self.proc.wait()
        for s in (self.proc.stdin, self.proc.stdout, self.proc.stderr):
            try:
                s.close()
            except Exception:
                pass
        shutil.rmtree(self.directory, ignore_errors=True)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
