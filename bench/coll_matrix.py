#!/usr/bin/env python
"""Time per cell of the collective matrix: AllReduce / AllGather / ReduceScatter / Broadcast / Reduce x
dtype x size (1 KB ... 1 GB in powers of 4), tuner's choice and every forced algorithm, next to NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        bench/coll_matrix.py [--max-mb 1024] [--dtypes fp32,bf16,fp16,int32] [--ops sum] [--out matrix.jsonl]

`size` is the per-rank message of AllReduce/Broadcast/Reduce and the total (n x per-rank part) of
AllGather/ReduceScatter.  Buffers are symmetric.  CUDA-event times, maximum over ranks.  Correctness of
every cell is covered by tests/test_gpu.py; this script only measures.
"""
from __future__ import annotations

import argparse
import json
import os
import struct
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mccl_b200 as mccl  # noqa: E402

DT = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16, "int32": torch.int32}
ROP = {"sum": dist.ReduceOp.SUM, "prod": dist.ReduceOp.PRODUCT, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "avg": dist.ReduceOp.AVG}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--dtypes", default="fp32,bf16,fp16,int32")
    ap.add_argument("--ops", default="sum")
    ap.add_argument("--colls", default="allreduce,allgather,reducescatter,broadcast,reduce")
    ap.add_argument("--algos", default="auto,ring,tree,oneshot,twoshot,nvls")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    lr = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    port = int(os.environ.get("MASTER_PORT", "29500")) + 41
    comm = mccl.Communicator(world, mccl.unique_id_from_env(os.environ.get("MASTER_ADDR", "127.0.0.1"), port), rank, transport="cuda")
    dist.init_process_group("nccl", device_id=dev)
    sink = open(args.out, "w") if (args.out and rank == 0) else None

    def hmax(v):
        return max(struct.unpack("d", b)[0] for b in comm.host_all_gather(struct.pack("d", v)))

    def timed(fn):
        fn(); fn()
        torch.cuda.synchronize(); comm.host_barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record(); torch.cuda.synchronize()
        return round(hmax(e0.elapsed_time(e1) / args.iters) * 1e3, 1)

    sizes = []
    b = 1024
    while b <= args.max_mb << 20:
        sizes.append(b); b *= 4
    wins = losses = 0
    for dname in args.dtypes.split(","):
        dt = DT[dname]
        es = torch.empty((), dtype=dt).element_size()
        for nbytes in sizes:
            n = max(nbytes // es // world * world, world)
            big = comm.empty(n, dt); small = comm.empty(n // world, dt)
            nb, ns = torch.empty(n, device=dev, dtype=dt), torch.empty(n // world, device=dev, dtype=dt)
            for t in (big, small, nb, ns):
                t.fill_(1)
            for op in args.ops.split(","):
                if op == "avg" and not dt.is_floating_point:
                    continue
                calls = {
                    "allreduce": (lambda: comm.all_reduce(big, op=op), lambda: dist.all_reduce(nb, op=ROP[op])),
                    "allgather": (lambda: comm.all_gather(small, big), lambda: dist.all_gather_into_tensor(nb, ns)),
                    "reducescatter": (lambda: comm.reduce_scatter(big, small, op=op), lambda: dist.reduce_scatter_tensor(ns, nb, op=ROP[op])),
                    "broadcast": (lambda: comm.broadcast(big, big, root=0), lambda: dist.broadcast(nb, 0)),
                    "reduce": (lambda: comm.reduce(big, big if rank == 0 else None, op=op, root=0), lambda: dist.reduce(nb, 0, op=ROP[op])),
                }
                for coll in args.colls.split(","):
                    mine, theirs = calls[coll]
                    row = {"coll": coll, "dtype": dname, "op": op, "bytes": n * es, "nccl_us": timed(theirs)}
                    for algo in args.algos.split(","):
                        with mccl.forced_algo(algo):
                            us = timed(mine)
                        ran = comm.last_algo
                        if algo == "auto":
                            row["auto_us"], row["auto_algo"] = us, ran
                        elif ran == algo:            # a forced algorithm that cannot run this cell falls back; skip the duplicate
                            row[f"{algo}_us"] = us
                        for t in (big, small):
                            t.fill_(1)
                    assert comm.async_error() == 0
                    if rank == 0:
                        wins += row["auto_us"] <= row["nccl_us"]; losses += row["auto_us"] > row["nccl_us"]
                        line = json.dumps(row)
                        print(line, flush=True)
                        if sink:
                            sink.write(line + "\n")
            comm.free_raw(big.data_ptr()); comm.free_raw(small.data_ptr())
            del big, small, nb, ns
    if rank == 0:
        print(json.dumps({"summary": "cells where the tuner's choice is at least as fast as NCCL", "wins": wins, "losses": losses}), flush=True)
    comm.finalize(); comm.destroy()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
