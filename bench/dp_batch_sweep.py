#!/usr/bin/env python
"""The reference's published experiment in its own shape: a data-parallel step = "compute on the batch + a 16 MB
gradient all-reduce", with the batch (bytes of data processed per step) swept from 64 MB to 32 GB, and

    speedup(batch) = T(1 GPU, whole batch) / T(N GPUs, batch / N each + all-reduce)

(README.md:55-57 and docs/perf-scaling.png of the reference: 1.0x / 1.7x / 2.1x / 2.7x / 2.9x of an ideal 3x at
64 MB / 256 MB / 1 GB / 4 GB / 32 GB on three machines).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench/dp_batch_sweep.py [--sizes-mb 64,256,1024,4096,32768] [--impl mccl|nccl]

The compute is a two-layer bf16 MLP (features x features twice = 16 MB of bf16 gradients at 2048 features),
forward and backward written out as matrix products over row chunks so that a 32 GB batch needs no more memory
than the batch itself; the gradients accumulate in one symmetric 16 MB buffer that is all-reduced (average) once
per step, followed by an SGD update.  Every rank first runs the whole batch alone (T1, no communication), then its
1/N share with the all-reduce (TN); times are CUDA-event times, maximum over ranks.  `--device cpu` runs the same
script on the tcp transport with small sizes (a check of the script, not a benchmark).
"""
from __future__ import annotations

import argparse
import json
import os
import struct
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mccl_b200 as mccl  # noqa: E402

PUBLISHED = {64: 1.0, 256: 1.7, 1024: 2.1, 4096: 2.7, 32768: 2.9}      # the reference, 3 machines


class Step:
    """One training step of the two-layer MLP on `rows` rows of this rank's data."""

    def __init__(self, features: int, dev, dtype, grads: torch.Tensor, chunk_rows: int):
        g = torch.Generator(device="cpu").manual_seed(7)
        f = features
        self.w1 = (torch.randn(f, f, generator=g) * f ** -0.5).to(device=dev, dtype=dtype)
        self.w2 = (torch.randn(f, f, generator=g) * f ** -0.5).to(device=dev, dtype=dtype)
        self.g1 = grads[: f * f].view(f, f)
        self.g2 = grads[f * f: 2 * f * f].view(f, f)
        self.grads = grads
        self.chunk = chunk_rows
        self.f = f

    def compute(self, x: torch.Tensor) -> None:
        """Forward + backward over the rows of x in chunks; the gradients of mean(y^2) over these rows are
        accumulated into the gradient buffer (which the caller has zeroed).  Averaging the buffers of equal shares
        over the ranks then gives the gradient of the whole batch."""
        scale = 2.0 / (x.shape[0] * self.f)
        for lo in range(0, x.shape[0], self.chunk):
            xc = x[lo: lo + self.chunk]
            h_pre = xc @ self.w1.t()
            h = torch.relu(h_pre)
            y = h @ self.w2.t()
            dy = y * scale
            self.g2.addmm_(dy.t(), h)
            dh = dy @ self.w2
            dh.mul_(h_pre > 0)
            self.g1.addmm_(dh.t(), xc)

    def update(self, lr: float = 1e-2) -> None:
        self.w1.add_(self.g1, alpha=-lr)
        self.w2.add_(self.g2, alpha=-lr)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", default="64,256,1024,4096,32768")
    ap.add_argument("--features", type=int, default=2048)
    ap.add_argument("--chunk-rows", type=int, default=65536)
    ap.add_argument("--impl", default="mccl", choices=["mccl", "nccl"])
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    lr_ = int(os.environ.get("LOCAL_RANK", rank))
    cuda = args.device == "cuda"
    if cuda:
        torch.cuda.set_device(lr_)
    dev = torch.device("cuda", lr_) if cuda else torch.device("cpu")
    dtype = torch.bfloat16 if cuda else torch.float32
    es = 2 if cuda else 4
    port = int(os.environ.get("MASTER_PORT", "29500")) + 37
    comm = None
    if world > 1 or args.impl == "mccl":
        comm = mccl.Communicator(world, mccl.unique_id_from_env(os.environ.get("MASTER_ADDR", "127.0.0.1"), port), rank,
                                 transport="cuda" if cuda else "tcp")
    if args.impl == "nccl" and world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    f = args.features
    n_grad = 2 * f * f
    grads = comm.empty(n_grad, dtype) if (cuda and comm is not None and world > 1 and args.impl == "mccl") else \
        torch.empty(n_grad, device=dev, dtype=dtype)
    step = Step(f, dev, dtype, grads, args.chunk_rows)

    def hmax(v: float) -> float:
        if comm is None:
            return v
        return max(struct.unpack("d", b)[0] for b in comm.host_all_gather(struct.pack("d", v)))

    def sync():
        if cuda:
            torch.cuda.synchronize()
        if comm is not None:
            comm.host_barrier()

    def all_reduce():
        if world == 1:
            return
        if args.impl == "mccl":
            comm.all_reduce(grads, op="avg")
        else:
            import torch.distributed as dist
            dist.all_reduce(grads, op=dist.ReduceOp.AVG)

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        sync()
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / steps
        else:
            t0 = time.perf_counter()
            for _ in range(steps):
                fn()
            ms = (time.perf_counter() - t0) * 1e3 / steps
        return hmax(ms)

    rows_out = []
    for mb in [int(s) for s in args.sizes_mb.split(",") if s]:
        rows = max(world, (mb << 20) // (f * es) // world * world)       # whole batch, divisible by the ranks
        share = rows // world
        # the data: this rank's copy of the whole batch for T1; its share is the slice [rank*share, (rank+1)*share)
        x = torch.empty(rows, f, device=dev, dtype=dtype)
        g = torch.Generator(device=dev).manual_seed(100)                   # same data on every rank
        for lo in range(0, rows, args.chunk_rows):
            x[lo: lo + args.chunk_rows].normal_(generator=g)
        steps = args.steps if mb <= 4096 else max(2, args.steps // 2)
        warm = args.warmup if mb <= 4096 else max(3, args.warmup // 2)

        def one_gpu():
            grads.zero_()
            step.compute(x)
            step.update()

        def n_gpus():
            grads.zero_()
            step.compute(x[rank * share:(rank + 1) * share])
            all_reduce()
            step.update()

        t1 = timed(one_gpu, steps, warm)
        tn = timed(n_gpus, steps, warm)
        ar = timed(all_reduce, 10, 3) if world > 1 else 0.0
        out = {"batch_mb": mb, "rows": rows, "features": f, "n_gpus": world, "impl": args.impl, "t1_ms": round(t1, 4),
               "tn_ms": round(tn, 4), "speedup": round(t1 / tn, 3), "ideal": world, "allreduce_ms": round(ar, 4),
               "grad_mbytes": round(n_grad * es / (1 << 20), 2), "reference_published_3_machines": PUBLISHED.get(mb)}
        rows_out.append(out)
        if rank == 0:
            print(json.dumps(out), flush=True)
        del x
        if cuda:
            torch.cuda.empty_cache()

    if args.device == "cpu" and world > 1:
        # check of the script: the averaged gradient of the shares equals the gradient of the whole batch
        rows = 8 * world
        gen = torch.Generator().manual_seed(5)
        x = torch.randn(rows, f, generator=gen)
        grads.zero_(); step.compute(x); whole = grads.clone()
        grads.zero_(); step.compute(x[rank * 8:(rank + 1) * 8]); comm.all_reduce(grads, op="avg")
        assert torch.allclose(grads, whole, atol=1e-5, rtol=1e-4), (grads - whole).abs().max().item()
        if rank == 0:
            print(json.dumps({"gradient_check": "ok"}), flush=True)
    if comm is not None:
        comm.finalize(); comm.destroy()
    if args.impl == "nccl" and world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
