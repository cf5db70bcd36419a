#!/usr/bin/env python
"""Small single-GPU cases of the library's own kernels, sized for profiling (inputs larger than the 126 MB
L2, a few hundred MB on the device, a handful of launches) and for quick CUDA-event timing.

    python bench/kernel_cases.py gemm   [--m 8192 --n 3584 --k 8192] [--launches 3]
    python bench/kernel_cases.py adamw  [--elems 67108864]
    python bench/kernel_cases.py sumsq  [--elems 268435456]
    python bench/kernel_cases.py copy   [--mbytes 512]      (staging copy kernel through a 1-rank communicator)
    python bench/kernel_cases.py emu    [--ranks 8 --mbytes 64 --algo twoshot|oneshot|ring|tree]
                                        (multi-rank all-reduce kernels with the ranks emulated on this one GPU)

Prints one JSON line with the CUDA-event time per launch and the achieved fraction of the measured peaks
(MEASURED_PEAKS.json next to the repository root if present, else 6451.8 GB/s and 1685 TFLOP/s).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return 6451.8, 1685.0, "recorded"


def timed(fn, launches, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    flush = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)
    total = 0.0
    for _ in range(launches):
        flush.zero_()                       # evict the previous launch's data from L2
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / launches


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "adamw", "sumsq", "copy", "emu"])
    ap.add_argument("--ranks", type=int, default=8)
    ap.add_argument("--algo", default="twoshot")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=3584)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--elems", type=int, default=0)
    ap.add_argument("--mbytes", type=int, default=512)
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--cublas", action="store_true", help="gemm: also time torch.matmul (cuBLAS) on the same operands")
    ap.add_argument("--two-sm", action="store_true", help="gemm: the form in which pairs of SMs share a 256-row tile")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    hbm, tflops, src = peaks()
    out = {"case": args.case, "peaks": src}
    if args.case == "gemm":
        from mccl_b200.ops import gemm as G
        x = torch.randn(args.m, args.k, device=dev).to(torch.bfloat16)
        w = (torch.randn(args.n, args.k, device=dev) * 0.02).to(torch.bfloat16)
        y = torch.empty(args.m, args.n, device=dev, dtype=torch.bfloat16)
        ms = timed(lambda: G.gemm(x, w, out=y, epilogue="silu", two_sm=args.two_sm), args.launches)
        fl = 2.0 * args.m * args.n * args.k
        out.update({"shape": [args.m, args.n, args.k], "two_sm": args.two_sm, "us": round(ms * 1e3, 1), "tflops": round(fl / ms / 1e9, 1),
                    "frac_of_cublas_peak": round(fl / ms / 1e9 / tflops, 3), "kernel_error": G.last_error()})
        if args.cublas:
            # the library GEMM on the same operands, timed the same way (no activation: it has none to fuse)
            ref_ms = timed(lambda: torch.matmul(x, w.t(), out=y), args.launches)
            out.update({"cublas_us": round(ref_ms * 1e3, 1), "cublas_tflops": round(fl / ref_ms / 1e9, 1),
                        "speedup_vs_cublas": round(ref_ms / ms, 3)})
    elif args.case == "adamw":
        from mccl_b200.ops.optim import fused_adamw_
        n = args.elems or (64 << 20)
        p = torch.zeros(n, device=dev, dtype=torch.bfloat16); g = torch.randn(n, device=dev).to(torch.bfloat16)
        m32 = torch.randn(n, device=dev); ea = torch.zeros(n, device=dev); es = torch.zeros(n, device=dev)
        ms = timed(lambda: fused_adamw_(p, m32, ea, es, g, lr=1e-3, step=1, zero_grad=False), args.launches)
        byts = n * (2 + 2 + 3 * 4 * 2)      # read grad, write param, read+write three fp32 arrays
        out.update({"elems": n, "us": round(ms * 1e3, 1), "gbs": round(byts / ms / 1e6, 1), "frac_of_copy_peak": round(byts / ms / 1e6 / hbm, 3)})
    elif args.case == "sumsq":
        from mccl_b200.ops.optim import scratch_floats, sum_squares_
        n = args.elems or (256 << 20)
        x = torch.randn(n, device=dev).to(torch.bfloat16)
        o = torch.zeros(1, device=dev); sc = torch.zeros(scratch_floats(n), device=dev)
        ms = timed(lambda: sum_squares_(x, o, sc), args.launches)
        out.update({"elems": n, "us": round(ms * 1e3, 1), "gbs": round(2 * n / ms / 1e6, 1), "frac_of_copy_peak": round(2 * n / ms / 1e6 / hbm, 3)})
    elif args.case == "emu":
        from mccl_b200 import emu
        n = (args.mbytes << 20) // 2
        xs = [torch.randn(n, device=dev).to(torch.bfloat16) for _ in range(args.ranks)]
        ms = timed(lambda: emu.all_reduce(xs, op="sum", algo=args.algo, ctas=16), args.launches)
        # local traffic of the emulation: every rank reads n-1 remote shards' worth twice and writes its buffer once
        out.update({"ranks": args.ranks, "bytes_per_rank": n * 2, "algo": args.algo, "us": round(ms * 1e3, 1),
                    "note": "all ranks share one GPU: times say nothing about NVLink"})
        emu.destroy()
    else:
        import mccl_b200 as mccl
        comm = mccl.Communicator(1, mccl.get_unique_id(), 0, transport="cuda")
        n = args.mbytes << 20
        a = torch.empty(n, device=dev, dtype=torch.uint8).random_(); b = torch.empty_like(a)
        ms = timed(lambda: comm.all_reduce(a, b, dtype=mccl.UINT8), args.launches)
        out.update({"bytes": n, "us": round(ms * 1e3, 1), "gbs": round(2 * n / ms / 1e6, 1), "frac_of_copy_peak": round(2 * n / ms / 1e6 / hbm, 3)})
        comm.finalize(); comm.destroy()
    print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
