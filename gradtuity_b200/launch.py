"""Process launcher: `python -m gradtuity_b200.launch --nproc N script.py [args...]`.

Same command line and environment contract as the reference's launcher (gradtuity/launch.py:25-103):
one worker per GPU with RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT and a shared
GRADTUITY_NCCL_UID_FILE; the first worker that exits non-zero takes its siblings down and its
code becomes the launcher's exit code.  Workers are polled, so a failure of any rank is seen at
once, not only after the ranks before it have finished.
"""
from __future__ import annotations

import argparse
import os
import random
import signal
import subprocess
import sys
import time


def worker_env(base: dict, rank: int, nproc: int, master_addr: str, master_port: int, uid_file: str) -> dict:
    env = dict(base)
    env.update({"MASTER_ADDR": master_addr, "MASTER_PORT": str(master_port), "WORLD_SIZE": str(nproc),
                "RANK": str(rank), "LOCAL_RANK": str(rank), "GRADTUITY_LAUNCHER": "1",
                "GRADTUITY_NCCL_UID_FILE": uid_file})
    return env


def run(nproc: int, script: str, script_args: list[str], master_addr: str = "127.0.0.1",
        master_port: int | None = None, poll_s: float = 0.05) -> int:
    if nproc <= 0:
        raise SystemExit("nproc must be > 0")
    port = master_port if master_port is not None else 29500 + random.randint(0, 1000)
    uid_file = f"/tmp/gradtuity_nccl_launch_{os.getpid()}.bin"
    try:
        os.remove(uid_file)
    except OSError:
        pass
    procs: list[subprocess.Popen] = []

    def shutdown() -> None:
        for p in procs:
            if p.poll() is None:
                try:
                    p.terminate()
                except Exception:
                    pass
        deadline = time.monotonic() + 1.0
        while time.monotonic() < deadline and any(p.poll() is None for p in procs):
            time.sleep(0.02)
        for p in procs:
            if p.poll() is None:
                try:
                    p.kill()
                except Exception:
                    pass

    def handle_sig(signum, frame) -> None:
        shutdown()
        raise SystemExit(128 + signum)

    old_int = signal.signal(signal.SIGINT, handle_sig)
    old_term = signal.signal(signal.SIGTERM, handle_sig)
    rc = 0
    try:
        for r in range(nproc):
            env = worker_env(os.environ.copy(), r, nproc, master_addr, port, uid_file)
            procs.append(subprocess.Popen([sys.executable, "-u", script] + list(script_args), env=env))
        pending = set(range(nproc))
        while pending:
            for i in list(pending):
                code = procs[i].poll()
                if code is None:
                    continue
                pending.discard(i)
                if code != 0 and rc == 0:
                    rc = code
            if rc != 0:
                break
            time.sleep(poll_s)
    finally:
        shutdown()
        signal.signal(signal.SIGINT, old_int)
        signal.signal(signal.SIGTERM, old_term)
        try:
            os.remove(uid_file)
        except OSError:
            pass
    return rc


def main() -> None:
    ap = argparse.ArgumentParser(prog="python -m gradtuity_b200.launch")
    ap.add_argument("--nproc", type=int, required=True, help="Number of worker processes")
    ap.add_argument("--master-addr", default="127.0.0.1", help="Rendezvous address")
    ap.add_argument("--master-port", type=int, default=None, help="Rendezvous port (default: auto)")
    ap.add_argument("script", help="Training script path")
    ap.add_argument("script_args", nargs=argparse.REMAINDER, help="Arguments passed to script")
    args = ap.parse_args()
    raise SystemExit(run(args.nproc, args.script, args.script_args, args.master_addr, args.master_port))


if __name__ == "__main__":
    main()
