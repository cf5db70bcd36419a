#!/usr/bin/env python
"""The collective matrix: AllReduce / AllGather / ReduceScatter / Broadcast / Reduce x {sum, prod, max, min, avg} x
{fp32, fp16, bf16, int32} x sizes 1 KB ... 1 GB in powers of 4, every result CHECKED against a reference computed
from the ranks' inputs (bit-exact for int32, within the dtype's tolerance for floats), the tuner's choice timed next
to NCCL and, on a subset of sizes, every forced algorithm next to the tuner's choice.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        bench/coll_matrix.py [--max-mb 1024] [--time-limit-s 600] [--out matrix.jsonl]

Inputs: element i of rank r is a fixed function of (r, i): uniform in [-1, 1] for floats, integers in [-1000, 1000]
for int32 (factors near 1 or of magnitude 1 for `prod`, so that products stay representable).  Any window of any
rank's input can therefore be rebuilt on every rank, and a cell is checked on windows at its start, middle and end
rather than on all of a 1 GB message.

`size` is the per-rank message of AllReduce / Broadcast / Reduce and the total (n x per-rank part) of AllGather /
ReduceScatter.  Buffers are symmetric.  CUDA-event times, maximum over ranks.  The cells run in three passes, most
important first, until `--time-limit-s` is spent: (1) every (collective, op, dtype) at four sizes, checked; (2) the
timing grid against NCCL (bf16 and fp32, sum, every size); (3) every forced algorithm at three sizes, checked.
The last line summarises cells run / exact / within tolerance / at least as fast as NCCL.
"""
from __future__ import annotations

import argparse
import json
import os
import struct
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mccl_b200 as mccl  # noqa: E402

DT = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16, "int32": torch.int32}
ROP = {"sum": dist.ReduceOp.SUM, "prod": dist.ReduceOp.PRODUCT, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "avg": dist.ReduceOp.AVG}
TOL = {torch.float32: 1e-5, torch.float16: 4e-3, torch.bfloat16: 3e-2}
REDUCING = ("allreduce", "reducescatter", "reduce")
WINDOW = 1 << 16            # elements per checked window


def values(r: int, lo: int, hi: int, dt, op: str, dev):
    """Elements [lo, hi) of rank r's input."""
    i = torch.arange(lo, hi, device=dev, dtype=torch.int64)
    h = (i * 2654435761 + (r + 1) * 40503 + (i >> 7) * 97) % 2001 - 1000          # integers in [-1000, 1000]
    if op == "prod":
        if dt.is_floating_point:
            return (1 + h.to(torch.float32) / 64000).to(dt)
        return torch.where(h % 2 == 0, 1, -1).to(dt)
    if dt.is_floating_point:
        return (h.to(torch.float32) / 1000).to(dt)
    return h.to(dt)


def reference(world: int, lo: int, hi: int, dt, op: str, dev):
    """The reduction of every rank's elements [lo, hi), in fp64 / exact integers."""
    st = torch.stack([values(r, lo, hi, dt, op, dev).double() if dt.is_floating_point else values(r, lo, hi, dt, op, dev).long()
                      for r in range(world)])
    if op in ("sum", "avg"):
        o = st.sum(0)
        if op == "avg":
            o = o / world if dt.is_floating_point else torch.div(o.to(dt), world, rounding_mode="trunc")
        return o
    if op == "prod":
        return st.prod(0)
    return st.max(0).values if op == "max" else st.min(0).values


def windows(n: int):
    """Up to three windows of at most WINDOW elements: start, middle, end."""
    if n <= 3 * WINDOW:
        return [(0, n)]
    mid = (n // 2) // 8 * 8
    return [(0, WINDOW), (mid, mid + WINDOW), (n - WINDOW, n)]


def grade(got, want, dt):
    """'exact', 'close' or 'WRONG' for one window."""
    if not dt.is_floating_point:
        return "exact" if torch.equal(got.long(), want.long()) else "WRONG"
    g, w = got.double(), want.double()
    if torch.equal(g, w.to(dt).double()):
        return "exact"
    err = ((g - w).abs() / (w.abs() + 1.0)).max().item()
    return "close" if err <= TOL[dt] else "WRONG"


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--time-limit-s", type=float, default=600.0, help="stop starting new cells after this many seconds")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--passes", default="1,2,3,4")
    ap.add_argument("--colls", default="allreduce,allgather,reducescatter,broadcast,reduce")
    ap.add_argument("--min-mb", type=float, default=0.0, help="skip cells smaller than this")
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
    t_start = time.time()
    stats = {"cells": 0, "exact": 0, "close": 0, "wrong": 0, "timed": 0, "at_or_above_nccl": 0, "algo_is_tuners_pick": 0, "forced_cells": 0}

    def hmax(v):
        return max(struct.unpack("d", b)[0] for b in comm.host_all_gather(struct.pack("d", v)))

    def out_of_time():
        # rank 0 decides, so that every rank stops at the same cell
        return struct.unpack("d", comm.host_all_gather(struct.pack("d", time.time() - t_start))[0])[0] > args.time_limit_s

    def timed(fn):
        fn(); fn()
        torch.cuda.synchronize(); comm.host_barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record(); torch.cuda.synchronize()
        return round(hmax(e0.elapsed_time(e1) / args.iters) * 1e3, 1)

    def fill(buf, r, op, base=0):
        n, step = buf.numel(), 1 << 24
        for lo in range(0, n, step):
            hi = min(n, lo + step)
            buf[lo:hi].copy_(values(r, base + lo, base + hi, buf.dtype, op, dev))

    bufs = {}

    def buffers(dname, n):
        key = (dname, n)
        if bufs.get("key") != key:
            for t in bufs.get("sym", []):
                comm.free_raw(t.data_ptr())
            bufs.clear()
            torch.cuda.empty_cache()
            dt = DT[dname]
            bufs["key"] = key
            bufs["sym"] = [comm.empty(n, dt), comm.empty(n // world, dt)]
            bufs["plain"] = [torch.empty(n, device=dev, dtype=dt), torch.empty(n // world, device=dev, dtype=dt)]
        return bufs["sym"] + bufs["plain"]

    def run_cell(coll, op, dname, nbytes, algo="auto", time_it=False, nccl=False):
        dt = DT[dname]
        es = torch.empty((), dtype=dt).element_size()
        n = max(nbytes // es // world * world, world)
        m = n // world
        big, small, nb, ns = buffers(dname, n)

        def prepare():
            if coll in ("allreduce", "reducescatter", "reduce"):
                fill(big, rank, op)
            elif coll == "allgather":
                fill(small, rank, op)
                big.fill_(7)
            else:
                if rank == 0:
                    fill(big, 0, op)
                else:
                    big.fill_(7)

        def call():
            if coll == "allreduce": comm.all_reduce(big, op=op)
            elif coll == "allgather": comm.all_gather(small, big)
            elif coll == "reducescatter": comm.reduce_scatter(big, small, op=op)
            elif coll == "broadcast": comm.broadcast(big, big, root=0)
            else: comm.reduce(big, big if rank == 0 else None, op=op, root=0)

        def nccl_call():
            if coll == "allreduce": dist.all_reduce(nb, op=ROP[op])
            elif coll == "allgather": dist.all_gather_into_tensor(nb, ns)
            elif coll == "reducescatter": dist.reduce_scatter_tensor(ns, nb, op=ROP[op])
            elif coll == "broadcast": dist.broadcast(nb, 0)
            else: dist.reduce(nb, 0, op=ROP[op])

        prepare()
        with mccl.forced_algo(algo):
            call()
            ran = comm.last_algo
            torch.cuda.synchronize()
            # ---- check this one call
            worst = "exact"
            order = {"exact": 0, "close": 1, "WRONG": 2}
            def note(v):
                nonlocal worst
                if order[v] > order[worst]: worst = v
            if coll == "allreduce" or (coll == "reduce" and rank == 0):
                for lo, hi in windows(n):
                    note(grade(big[lo:hi], reference(world, lo, hi, dt, op, dev), dt))
            elif coll == "reducescatter":
                for lo, hi in windows(m):
                    note(grade(small[lo:hi], reference(world, rank * m + lo, rank * m + hi, dt, op, dev), dt))
            elif coll == "allgather":
                for p in sorted({0, world // 2, world - 1}):
                    w = min(m, WINDOW)
                    note(grade(big[p * m:p * m + w], values(p, 0, w, dt, op, dev), dt))
                    note(grade(big[(p + 1) * m - w:(p + 1) * m], values(p, m - w, m, dt, op, dev), dt))
            elif coll == "broadcast":
                for lo, hi in windows(n):
                    note(grade(big[lo:hi], values(0, lo, hi, dt, op, dev), dt))
            if comm.async_error() != 0:
                worst = "WRONG"
            worst = max((b.decode() for b in comm.host_all_gather(worst.encode().ljust(5))), key=lambda v: order[v.strip()]).strip()
            row = {"coll": coll, "dtype": dname, "op": op, "bytes": n * es, "algo": algo, "ran": ran, "check": worst}
            if algo != "auto" and ran != algo and not time_it:
                pass
            if time_it:
                prepare()
                row["us"] = timed(call)
        if nccl:
            nb.fill_(1); ns.fill_(1)
            row["nccl_us"] = timed(nccl_call)
        stats["cells"] += 1
        stats["exact"] += worst == "exact"; stats["close"] += worst == "close"; stats["wrong"] += worst == "WRONG"
        if algo == "auto":
            # did the launcher run what the planner announced for this call, or fall back to something else?
            pick = comm.pick_algo(coll, n * es, mccl.comm._torch_dtypes()[dt], op)
            row["tuner"] = pick
            stats["algo_is_tuners_pick"] += ran == pick
        else:
            stats["forced_cells"] += ran == algo
        if "us" in row and "nccl_us" in row:
            stats["timed"] += 1
            stats["at_or_above_nccl"] += row["us"] <= row["nccl_us"]
        if rank == 0:
            line = json.dumps(row)
            print(line, flush=True)
            if sink:
                sink.write(line + "\n"); sink.flush()

    sizes = []
    b = 1024
    while b <= args.max_mb << 20:
        sizes.append(b); b *= 4
    colls = tuple(c for c in ("allreduce", "allgather", "reducescatter", "broadcast", "reduce") if c in args.colls.split(","))
    sizes = [s_ for s_ in sizes if s_ >= args.min_mb * (1 << 20)]
    ops_of = lambda coll: ("sum", "prod", "max", "min", "avg") if coll in REDUCING else ("sum",)
    passes = set(args.passes.split(","))
    done = set()
    stopped = False

    def cells_pass1():
        for dname in DT:
            for nbytes in [s for s in sizes if s in (1 << 10, 1 << 16, 1 << 22, 1 << 26)]:
                for coll in colls:
                    for op in ops_of(coll):
                        yield coll, op, dname, nbytes, "auto", False, False

    def cells_pass2():
        for dname in ("bf16", "fp32"):
            for nbytes in sizes:
                for coll in colls:
                    yield coll, "sum", dname, nbytes, "auto", True, True

    def cells_pass3():
        for dname in ("bf16", "int32"):
            for nbytes in [s for s in sizes if s in (1 << 16, 1 << 22, 1 << 26)]:
                for coll in colls:
                    for algo in ("ring", "tree", "oneshot", "twoshot", "nvls"):
                        yield coll, "sum", dname, nbytes, algo, True, False

    def cells_pass4():
        for dname in DT:
            for nbytes in sizes:
                for coll in colls:
                    for op in ops_of(coll):
                        yield coll, op, dname, nbytes, "auto", False, False

    for name, gen in (("1", cells_pass1), ("2", cells_pass2), ("3", cells_pass3), ("4", cells_pass4)):
        if name not in passes or stopped:
            continue
        for cell in gen():
            key = cell[:5]
            if key in done and not cell[5]:
                continue
            if out_of_time():
                stopped = True
                break
            run_cell(*cell)
            done.add(key)
    for t in bufs.get("sym", []):
        comm.free_raw(t.data_ptr())
    if rank == 0:
        stats["stopped_by_time_limit"] = stopped
        stats["seconds"] = round(time.time() - t_start, 1)
        stats["world"] = world
        line = json.dumps({"summary": stats})
        print(line, flush=True)
        if sink:
            sink.write(line + "\n")
    comm.finalize(); comm.destroy()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
