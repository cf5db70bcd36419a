"""Expert-parallel token exchange: the fused scatter / gather kernels against the packed form over NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench/moe_exchange.py [--tokens 8192] [--hidden 7168] [--experts-per-rank 2] [--capacity-factor 1.0]

Every rank routes `tokens` rows of `hidden` bf16 values to n x experts_per_rank experts (top-1).  With the default
capacity factor 1.0 the routing is an exact balance (a random permutation), so the packed form sends no padding
and both forms move the same bytes; with a larger factor the routing is random and the packed form also sends its
empty slots, as a fixed-capacity implementation does.

  fused     dispatch = one `mcclMoeScatter` (rows go from the activation tensor straight into their slot on the
            expert's rank); combine = one `mcclMoeGather` (rows come back scaled by the gate)
  packed    dispatch = zero a send buffer, index_copy the rows into it, `all_to_all_single` of equal blocks;
            combine = `all_to_all_single` back, index_select by slot, multiply by the gate

Both produce the same [ranks, experts_per_rank, capacity, hidden] buffer and the same [tokens, hidden] result; the
script compares them exactly before timing.  Times are CUDA events on the launching stream, maximum over ranks; the
buffers (117 MB per rank and direction at the defaults) do not fit next to each other in L2 with the activations.
Prints one JSON line on rank 0.
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
import mccl_b200 as mccl                                           # noqa: E402
from mccl_b200.ops import moe                                      # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts-per-rank", type=int, default=2)
    ap.add_argument("--capacity-factor", type=float, default=1.0)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    lr = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    port = int(os.environ.get("MASTER_PORT", "29500")) + 37
    comm = mccl.Communicator(world, mccl.unique_id_from_env(os.environ.get("MASTER_ADDR", "127.0.0.1"), port), rank, transport="cuda")
    dist.init_process_group("nccl", device_id=dev)

    T, d, e = args.tokens, args.hidden, args.experts_per_rank
    experts = world * e
    g = torch.Generator(device="cpu").manual_seed(1234 + rank)
    if args.capacity_factor <= 1.0:
        if T % experts:
            raise SystemExit("--tokens must be a multiple of the number of experts for the balanced routing")
        cap = T // experts
        flat = torch.randperm(T, generator=g).to(torch.int32)      # slot k of expert j is flat value j * cap + k
    else:
        cap = int(T / experts * args.capacity_factor + 0.999)
        expert = torch.randint(0, experts, (T,), generator=g)
        slot = torch.zeros(T, dtype=torch.long)
        fill = [0] * experts
        for t in range(T):
            j = int(expert[t]); slot[t] = fill[j]; fill[j] += 1
        flat = torch.where(slot < cap, expert * cap + slot, torch.full_like(slot, -1)).to(torch.int32)
    flat = flat.to(dev)
    x = torch.randn(T, d, generator=g).to(dev, torch.bfloat16)
    gate = torch.rand(T, generator=g).to(dev)
    buf = moe.ExchangeBuffer(comm, e, cap, d, torch.bfloat16)

    # ---- packed form over NCCL
    send = torch.empty(world, e, cap, d, device=dev, dtype=torch.bfloat16)
    recv = torch.empty_like(send)
    back = torch.empty_like(send)
    keep = (flat >= 0).nonzero().squeeze(1)
    flat_kept = flat[keep].long()

    def packed_dispatch():
        send.zero_()
        send.view(-1, d).index_copy_(0, flat_kept, x[keep] if keep.numel() != T else x)
        dist.all_to_all_single(recv.view(world, -1), send.view(world, -1))
        return recv

    def packed_combine(expert_out):
        dist.all_to_all_single(back.view(world, -1), expert_out.view(world, -1))
        rows = back.view(-1, d).index_select(0, flat.clamp(min=0).long())
        return (rows.float() * (gate * (flat >= 0)).unsqueeze(1)).to(torch.bfloat16)

    def fused_dispatch():
        moe._scatter(buf, x, flat, None)
        return buf.data

    def fused_combine():
        return moe._gather(buf, flat, gate, T)

    # ---- same results
    want = packed_dispatch().clone()
    got = fused_dispatch()
    torch.cuda.synchronize()
    same_dispatch = bool(torch.equal(want, got))
    y_want = packed_combine(want)
    y_got = fused_combine()                                        # the buffer still holds the dispatched rows
    torch.cuda.synchronize()
    combine_err = float((y_want.float() - y_got.float()).abs().max())

    def hmax(v: float) -> float:
        return max(struct.unpack("d", b)[0] for b in comm.host_all_gather(struct.pack("d", v)))

    def timed(fn) -> float:
        for _ in range(3):
            fn()
        torch.cuda.synchronize(); comm.host_barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record(); torch.cuda.synchronize()
        return hmax(e0.elapsed_time(e1) / args.iters * 1e3)       # us

    out = {
        "case": "moe_exchange", "n_gpus": world, "tokens_per_rank": T, "hidden": d, "experts": experts, "capacity": cap,
        "dropped": int((flat < 0).sum()), "dtype": "bf16", "same_dispatch": same_dispatch, "combine_max_abs_err": combine_err,
        "fused_dispatch_us": round(timed(fused_dispatch), 1),
        "packed_dispatch_us": round(timed(packed_dispatch), 1),
        "fused_combine_us": round(timed(fused_combine), 1),
        "packed_combine_us": round(timed(lambda: packed_combine(want)), 1),
        "api_dispatch_us": None, "api_combine_us": None,
    }
    gbuf = moe.ExchangeBuffer(comm, e, cap, d, torch.bfloat16)
    with torch.no_grad():
        out["api_dispatch_us"] = round(timed(lambda: moe.dispatch(x, flat, buf, gbuf)), 1)
        out["api_combine_us"] = round(timed(lambda: moe.combine(want, flat, gate, buf, gbuf)), 1)
    sent = int((flat >= 0).sum()) * d * 2 * (world - 1) / world      # bytes that leave this GPU, expected
    out["bytes_over_nvlink_per_rank"] = int(sent)
    for k in ("fused_dispatch", "packed_dispatch", "fused_combine", "packed_combine"):
        out[k + "_gbs"] = round(sent / out[k + "_us"] / 1e3, 1)
    out["dispatch_speedup"] = round(out["packed_dispatch_us"] / out["fused_dispatch_us"], 3)
    out["combine_speedup"] = round(out["packed_combine_us"] / out["fused_combine_us"], 3)
    out["async_error"] = comm.async_error()
    if rank == 0:
        print(json.dumps(out), flush=True)
    comm.finalize(); comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
