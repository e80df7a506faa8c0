"""Process supervisor: run N copies of a command as one unit.

    python -m miles_b200.orchestration.workers.supervisor --nproc 8 [--env-rank RANK] -- python train.py …

Every child gets `RANK` / `LOCAL_RANK` / `WORLD_SIZE` (names configurable); SIGTERM / SIGINT received by the supervisor
are forwarded to the children; as soon as ONE child exits non-zero the others are ended (a lone failed rank would
otherwise leave its peers blocked in a collective); the exit code is the first failing child's (128 + signal number
when it died from a signal), 0 when all succeeded.

Reference: miles/utils/workers/process_supervisor.py:24-152, process_trampoline.py:1-33.
"""
from __future__ import annotations

import argparse
import os
import signal
import subprocess
import sys
import time


def exit_code_of(returncode: int) -> int:
    return 128 - returncode if returncode < 0 else returncode


def supervise(cmd: list[str], nproc: int, env_rank: str = "RANK", env_local_rank: str = "LOCAL_RANK",
              env_world: str = "WORLD_SIZE", extra_env: dict | None = None, grace: float = 15.0, poll: float = 0.1) -> int:
    procs: list[subprocess.Popen] = []
    for r in range(nproc):
        env = {**os.environ, **(extra_env or {}), env_rank: str(r), env_local_rank: str(r), env_world: str(nproc)}
        procs.append(subprocess.Popen(cmd, env=env, start_new_session=True))
    got_signal: list[int] = []

    def forward(signum, _frame):
        got_signal.append(signum)
        for p in procs:
            if p.poll() is None:
                p.send_signal(signum)

    old = {s: signal.signal(s, forward) for s in (signal.SIGTERM, signal.SIGINT)}
    first_bad = None
    try:
        while any(p.poll() is None for p in procs):
            for p in procs:
                rc = p.poll()
                if rc is not None and rc != 0 and first_bad is None:
                    first_bad = rc
            if first_bad is not None:
                break
            time.sleep(poll)
        if first_bad is not None:
            for p in procs:
                if p.poll() is None:
                    p.terminate()
            end = time.monotonic() + grace
            for p in procs:
                try:
                    p.wait(timeout=max(0.0, end - time.monotonic()))
                except subprocess.TimeoutExpired:
                    p.kill()
                    p.wait()
    finally:
        for s, h in old.items():
            signal.signal(s, h)
    if first_bad is None:
        first_bad = next((p.returncode for p in procs if p.returncode), 0)
    return exit_code_of(first_bad)


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    cmd: list[str] = []
    if "--" in argv:
        i = argv.index("--")
        argv, cmd = argv[:i], argv[i + 1:]
    p = argparse.ArgumentParser(prog="miles_b200 supervisor")
    p.add_argument("--nproc", type=int, default=1)
    p.add_argument("--env-rank", default="RANK")
    p.add_argument("--env-local-rank", default="LOCAL_RANK")
    p.add_argument("--env-world", default="WORLD_SIZE")
    p.add_argument("--grace", type=float, default=15.0)
    a = p.parse_args(argv)
    assert cmd, "give the command after --"
    return supervise(cmd, a.nproc, a.env_rank, a.env_local_rank, a.env_world, grace=a.grace)


if __name__ == "__main__":
    sys.exit(main())
