"""Run one scenario of tests/_worker.py as `world` processes on this host and collect their verdicts."""
from __future__ import annotations

import json
import os
import socket
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def run_ranks(world: int, scenario: str, env: dict | None = None, timeout: int = 180, args: dict | None = None,
              per_rank_env: dict | None = None, worker: str = "_worker.py"):
    port = free_port()
    procs = []
    for r in range(world):
        e = dict(os.environ)
        e.update({"MCCL_TEST_RANK": str(r), "MCCL_TEST_WORLD": str(world), "MCCL_TEST_PORT": str(port),
                  "MCCL_TEST_ARGS": json.dumps(args or {}), "PYTHONPATH": ROOT + os.pathsep + e.get("PYTHONPATH", "")})
        e.update(env or {})
        e.update((per_rank_env or {}).get(r, {}))
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, worker), scenario], env=e,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    results = []
    for r, p in enumerate(procs):
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()          # the exact children started above
            out, _ = p.communicate()
            results.append((r, -9, out))
            continue
        results.append((r, p.returncode, out))
    return results


def assert_all_ok(results):
    bad = [(r, rc, out[-3000:]) for r, rc, out in results if rc != 0]
    assert not bad, "\n".join(f"--- rank {r} exit {rc}\n{out}" for r, rc, out in bad)
