#!/usr/bin/env python
"""All-reduce bus bandwidth of this library next to NCCL on the same GPUs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench/allreduce_sweep.py [--sizes-mb 64,256,1024,4096,32768] [--dtypes bf16,fp32] [--ops sum,avg] [--algos auto]

Buffers are symmetric (mcclMemAlloc) and reduced in place (`--plain` adds the same call on an ordinary torch
tensor, which is staged); values ~N(0,1) seeded by rank.  Every number is
timed on the device with CUDA events after warm-up and is the maximum over ranks.  bus GB/s =
bytes / time * 2(n-1)/n.  Rank 0 prints one JSON line per (size, dtype, op).
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


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", default="64,256,1024,4096,32768")
    ap.add_argument("--sizes-bytes", default="", help="explicit byte sizes (overrides --sizes-mb)")
    ap.add_argument("--dtypes", default="bf16,fp32")
    ap.add_argument("--ops", default="sum,avg")
    ap.add_argument("--algos", default="auto", help="comma list of auto,oneshot,twoshot,nvls,ring,tree")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--ctas-list", default="", help="tuning aid: run every algorithm with each of these exact CTA counts")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--plain", action="store_true",
                    help="also time the call on an ordinary torch tensor (staged through the communicator's symmetric scratch)")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    lr = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    port = int(os.environ.get("MASTER_PORT", "29500")) + 31
    comm = mccl.Communicator(world, mccl.unique_id_from_env(os.environ.get("MASTER_ADDR", "127.0.0.1"), port), rank, transport="cuda")
    if args.ctas:
        comm.set_max_ctas(args.ctas)
    if not args.no_nccl:
        dist.init_process_group("nccl", device_id=dev)

    def hmax(v):
        return max(struct.unpack("d", b)[0] for b in comm.host_all_gather(struct.pack("d", v)))

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(); comm.host_barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record(); torch.cuda.synchronize()
        return hmax(e0.elapsed_time(e1) / iters)

    sizes = [int(s) for s in args.sizes_bytes.split(",") if s] or [int(float(s) * (1 << 20)) for s in args.sizes_mb.split(",")]
    dts = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}
    k = 2 * (world - 1) / world
    for nbytes in sizes:
        for dname in args.dtypes.split(","):
            dt = dts[dname]
            n = nbytes // torch.empty((), dtype=dt).element_size()
            iters = max(3, min(args.iters, int(2e10 // max(nbytes, 1)) or 3))
            g = torch.Generator(device="cuda").manual_seed(rank)
            buf = comm.empty(n, dt)
            buf.normal_(generator=g)
            ref = None if args.no_nccl else torch.empty(n, device=dev, dtype=dt).normal_(generator=g)
            for op in args.ops.split(","):
                row = {"bytes": nbytes, "dtype": dname, "op": op, "n_gpus": world}
                if ref is not None:
                    rop = dist.ReduceOp.SUM if op == "sum" else dist.ReduceOp.AVG
                    ms = timed(lambda: dist.all_reduce(ref, op=rop), iters)
                    row["nccl_us"] = round(ms * 1e3, 1); row["nccl_busbw"] = round(nbytes / ms / 1e6 * k, 1)
                for ctas in [int(c) for c in args.ctas_list.split(",") if c] or [0]:
                    comm.set_ctas(ctas)
                    tag = f"@{ctas}" if ctas else ""
                    for algo in args.algos.split(","):
                        with mccl.forced_algo(algo):
                            ms = timed(lambda: comm.all_reduce(buf, op=op), iters)
                        row[f"mccl_{algo}{tag}_us"] = round(ms * 1e3, 1)
                        row[f"mccl_{algo}{tag}_busbw"] = round(nbytes / ms / 1e6 * k, 1)
                        if not ctas:
                            row[f"mccl_{algo}_ran"] = comm.last_algo
                        buf.normal_(generator=g)      # avg/sum in place would otherwise shrink or overflow the values
                comm.set_ctas(0)
                if args.plain:
                    plain = ref if ref is not None else torch.empty(n, device=dev, dtype=dt)
                    plain.normal_(generator=g)
                    ms = timed(lambda: comm.all_reduce(plain, op=op), iters)
                    row["mccl_plain_us"] = round(ms * 1e3, 1)
                    row["mccl_plain_busbw"] = round(nbytes / ms / 1e6 * k, 1)
                    row["plain_vs_symmetric"] = round(row["mccl_auto_us"] / (ms * 1e3), 3) if "mccl_auto_us" in row else None
                assert comm.async_error() == 0
                if rank == 0:
                    print(json.dumps(row), flush=True)
            comm.free_raw(buf.data_ptr())
            del buf, ref
            torch.cuda.empty_cache()
    comm.finalize(); comm.destroy()
    if not args.no_nccl:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
