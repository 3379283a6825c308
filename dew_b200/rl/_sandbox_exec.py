"""Apply process limits, then exec the program: run as ``python -I _sandbox_exec.py <cpu seconds> <memory bytes> <files> argv...``.

A launcher of its own (rather than a ``preexec_fn``) because a threaded parent must not run Python between fork and exec.
Reference: src/dew/rl/_sandbox_exec.py.
"""
import os
import resource
import sys


def main() -> None:
    cpu, memory, files = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    argv = sys.argv[4:]
    if cpu > 0:
        resource.setrlimit(resource.RLIMIT_CPU, (cpu, cpu + 1))
    if memory > 0:
        resource.setrlimit(resource.RLIMIT_AS, (memory, memory))
    if files > 0:
        resource.setrlimit(resource.RLIMIT_FSIZE, (files, files))
    resource.setrlimit(resource.RLIMIT_CORE, (0, 0))
    os.execvp(argv[0], argv)


if __name__ == "__main__":
    main()
