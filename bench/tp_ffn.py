#!/usr/bin/env python
"""Tensor-parallel Llama-style FFN: fused all-gather -> up-GEMM -> SiLU and down-GEMM -> reduce-scatter
(this library's tcgen05 kernels with the communication inside) next to NCCL all-gather / reduce-scatter +
cuBLAS on the same GPUs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        bench/tp_ffn.py [--tokens 8192 --hidden 8192 --ffn 28672] [--tp 8|4]

--tp 4 on 8 GPUs splits the communicator into two TP=4 groups (mcclCommSplit), the TP=4 x DP=2 layout.
Activations ~N(0,1), weights ~N(0,0.02), bf16.  Times are CUDA-event times, maximum over ranks.  The
roofline of each fused op is the slower of its FLOPs at the measured cuBLAS rate and its NVLink bytes at
the measured 770 GB/s per direction.  Rank 0 prints one JSON line.
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
from mccl_b200.ops import gemm as G  # noqa: E402
from mccl_b200.parallel.tp import TensorParallelFFN  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--tp", type=int, default=0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--peak-tflops", type=float, default=1685.0)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    lr = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    port = int(os.environ.get("MASTER_PORT", "29500")) + 37
    world_comm = mccl.Communicator(world, mccl.unique_id_from_env(os.environ.get("MASTER_ADDR", "127.0.0.1"), port), rank, transport="cuda")
    dist.init_process_group("nccl", device_id=dev)
    tp = args.tp or world
    comm, group = world_comm, None
    if tp != world:
        comm = world_comm.split(rank // tp, rank)
        groups = [dist.new_group(list(range(g * tp, (g + 1) * tp))) for g in range(world // tp)]
        group = groups[rank // tp]
    n, r = comm.size, comm.rank
    M, H, F = args.tokens, args.hidden, args.ffn
    g = torch.Generator(device="cuda").manual_seed(rank)
    x_shard = torch.randn(M // n, H, generator=g, device=dev).to(torch.bfloat16)
    w_up = (torch.randn(F // n, H, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    w_down = (torch.randn(H, F // n, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    layer = TensorParallelFFN(comm, M, H, F, w_up, w_down)
    layer.x_shard.copy_(x_shard)

    def hmax(v):
        return max(struct.unpack("d", b)[0] for b in world_comm.host_all_gather(struct.pack("d", v)))

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(); world_comm.host_barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record(); torch.cuda.synchronize()
        return hmax(e0.elapsed_time(e1) / iters)

    lib = G._lib()
    import ctypes as C
    h = C.c_void_p(comm.handle)
    s = lambda: C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def fused_up():
        mccl._lib.check(lib.mcclTpAllGatherGemm(h, layer.x_shard.data_ptr(), layer.x_full.data_ptr(), w_up.data_ptr(), layer.h.data_ptr(),
                                                layer.ag_flags.data_ptr(), M, F // n, H, 1, s()))

    def fused_down():
        layer.calls += 1
        mccl._lib.check(lib.mcclTpGemmReduceScatter(h, layer.h.data_ptr(), w_down.data_ptr(), layer.partial.data_ptr(),
                                                    layer.flags.data_ptr(), layer.out.data_ptr(), layer.accum.data_ptr(), M, H, F // n, layer.calls, s()))

    # NCCL + cuBLAS baseline on the same shapes
    x_full = torch.empty(M, H, device=dev, dtype=torch.bfloat16)
    hb = torch.empty(M, F // n, device=dev, dtype=torch.bfloat16)
    yb = torch.empty(M, H, device=dev, dtype=torch.bfloat16)
    ob = torch.empty(M // n, H, device=dev, dtype=torch.bfloat16)

    def base_up():
        dist.all_gather_into_tensor(x_full, x_shard, group=group)
        torch.matmul(x_full, w_up.t(), out=hb)
        torch.nn.functional.silu(hb, inplace=True)

    def base_down():
        torch.matmul(hb, w_down.t(), out=yb)
        dist.reduce_scatter_tensor(ob, yb, group=group)

    res = {"n_gpus": world, "tp": n, "tokens": M, "hidden": H, "ffn": F}
    res["fused_up_us"] = round(timed(fused_up, args.iters) * 1e3, 1)
    res["fused_down_us"] = round(timed(fused_down, args.iters) * 1e3, 1)
    res["fused_ffn_us"] = round(timed(lambda: (fused_up(), fused_down()), args.iters) * 1e3, 1)
    res["nccl_cublas_up_us"] = round(timed(base_up, args.iters) * 1e3, 1)
    res["nccl_cublas_down_us"] = round(timed(base_down, args.iters) * 1e3, 1)
    res["nccl_cublas_ffn_us"] = round(timed(lambda: (base_up(), base_down()), args.iters) * 1e3, 1)
    res["cublas_up_gemm_only_us"] = round(timed(lambda: torch.matmul(x_full, w_up.t(), out=hb), args.iters) * 1e3, 1)
    res["mccl_up_gemm_only_us"] = round(timed(lambda: G.gemm(x_full, w_up, out=hb, epilogue="silu"), args.iters) * 1e3, 1)
    flops = 2.0 * M * (F // n) * H
    link_bytes = (n - 1) / n * M * H * 2
    roof_us = max(flops / (args.peak_tflops * 1e12), link_bytes / (args.link_gbs * 1e9)) * 1e6
    res["roofline_us_per_op"] = round(roof_us, 1)
    res["fused_up_frac_of_roofline"] = round(roof_us / res["fused_up_us"], 3)
    res["fused_down_frac_of_roofline"] = round(roof_us / res["fused_down_us"], 3)
    res["speedup_vs_nccl_cublas"] = round(res["nccl_cublas_ffn_us"] / res["fused_ffn_us"], 3)
    res["kernel_errors"] = G.last_error()
    # numerics of the fused pair against the baseline pair
    fused_up(); fused_down(); base_up(); base_down(); torch.cuda.synchronize()
    res["max_abs_diff_vs_baseline"] = round((layer.out.float() - ob.float()).abs().max().item(), 4)
    res["out_abs_max"] = round(ob.float().abs().max().item(), 3)
    if rank == 0:
        print(json.dumps(res), flush=True)
    if comm is not world_comm:
        comm.finalize(); comm.destroy()
    world_comm.finalize(); world_comm.destroy()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
