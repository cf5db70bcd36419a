#!/usr/bin/env python
"""CPU plumbing benchmark: `--world` processes on loopback over the tcp transport, 1 Mi fp32 per rank
~U[-1,1] seeded by rank; times sum all-reduce, all-gather, reduce-scatter, broadcast(root 0), reduce(root 1)
and a split, checks every result against numpy, and prints one JSON line (wall-clock ms, maximum over ranks,
best of `--iters`).

    python bench/cpu_plumbing.py [--world 2] [--count 1048576] [--iters 5]
"""
from __future__ import annotations

import argparse
import json
import multiprocessing as mp
import os
import socket
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rank_main(rank, world, port, count, iters, q):
    import mccl_b200 as mccl
    comm = mccl.Communicator(world, mccl.unique_id_from_env("127.0.0.1", port), rank, transport="tcp")
    xs = [np.random.default_rng(r).uniform(-1, 1, count).astype(np.float32) for r in range(world)]
    x, ref = xs[rank], np.sum(xs, axis=0, dtype=np.float64)
    blk = count // world
    res, ok = {}, True

    def best(fn):
        t = []
        for _ in range(iters):
            comm.host_barrier()
            t0 = time.perf_counter(); fn(); t.append((time.perf_counter() - t0) * 1e3)
        return min(t)

    for algo in ("auto", "ring", "tree", "oneshot"):
        with mccl.forced_algo(algo):
            out = np.empty_like(x)
            res[f"allreduce_{algo}_ms"] = best(lambda: comm.all_reduce(x, out))
            ok &= bool(np.max(np.abs(out - ref) / (np.abs(ref) + 1.0)) < 1e-6)
    g = np.empty(count * world, np.float32)
    res["allgather_ms"] = best(lambda: comm.all_gather(x, g)); ok &= np.array_equal(g, np.concatenate(xs))
    rs = np.empty(blk, np.float32)
    res["reducescatter_ms"] = best(lambda: comm.reduce_scatter(x[:blk * world], rs))
    ok &= bool(np.max(np.abs(rs - ref[rank * blk:(rank + 1) * blk])) < 1e-5)
    b = x.copy() if rank == 0 else np.zeros_like(x)
    res["broadcast_ms"] = best(lambda: comm.broadcast(b if rank == 0 else None, b, root=0)); ok &= np.array_equal(b, xs[0])
    root = 1 % world
    rd = np.empty_like(x) if rank == root else None
    res["reduce_ms"] = best(lambda: comm.reduce(x, rd, root=root))
    if rank == root:
        ok &= bool(np.max(np.abs(rd - ref) / (np.abs(ref) + 1.0)) < 1e-6)
    t0 = time.perf_counter(); sub = comm.split(rank, 0); res["split_ms"] = (time.perf_counter() - t0) * 1e3
    ok &= sub.size == 1
    sub.destroy()
    comm.finalize(); comm.destroy()
    q.put((rank, ok, res))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--count", type=int, default=1 << 20)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=rank_main, args=(r, a.world, port, a.count, a.iters, q)) for r in range(a.world)]
    [p.start() for p in ps]
    got = [q.get(timeout=300) for _ in ps]
    [p.join() for p in ps]
    out = {"world": a.world, "count": a.count, "dtype": "fp32", "transport": "tcp (loopback)", "all_match_numpy": all(g[1] for g in got)}
    for key in got[0][2]:
        out[key] = round(max(g[2][key] for g in got), 2)
    print(json.dumps(out))
    return 0 if out["all_match_numpy"] else 1


if __name__ == "__main__":
    sys.exit(main())
