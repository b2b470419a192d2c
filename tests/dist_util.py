"""Launch the multi-process worker: one child per rank, loopback rendezvous, hard deadline, children killed by
exact PID on failure."""
import json
import os
import socket
import subprocess
import sys
import time


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(scenario: str, world: int, tmp_path, timeout: float = 240.0, extra_env=None):
    port = free_port()
    out = str(tmp_path / f"{scenario}.json")
    procs = []
    worker = os.path.join(os.path.dirname(__file__), "dist_worker.py")
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2")
        env.update(extra_env or {})
        procs.append(subprocess.Popen([sys.executable, worker, scenario, out], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    deadline = time.time() + timeout
    try:
        for p in procs:
            left = max(1.0, deadline - time.time())
            p.wait(timeout=left)
    except subprocess.TimeoutExpired:
        for p in procs:
            if p.poll() is None:
                p.kill()
        raise AssertionError(f"{scenario}: ranks did not finish within {timeout}s")
    logs = [p.stdout.read() for p in procs]
    for rank, p in enumerate(procs):
        assert p.returncode == 0, f"rank {rank} failed:\n{logs[rank][-3000:]}"
    results = []
    for rank in range(world):
        with open(f"{out}.{rank}") as f:
            results.append(json.load(f))
    return results
