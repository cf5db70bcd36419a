"""Send / Recv bandwidth: a ring exchange (every rank sends to rank + 1 and receives from rank - 1 in one group) and
an all-pairs exchange (every rank sends a block to every other rank, the grouped form of an all-to-all), this
library against NCCL's `batch_isend_irecv` on the same tensors.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench/sendrecv.py [--sizes-kb 64,1024,16384,262144]

Messages are ordinary torch tensors (Send / Recv goes through the per-peer FIFO in the receiver's control segment,
whatever memory the user's buffers are in).  The received bytes are compared with what the sender holds before the
timing.  CUDA events on the launching stream, 3 warm-ups + `--iters` timed groups, maximum over ranks.  One JSON
line per size on rank 0; `*_gbs` is bytes received per GPU and second.
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-kb", default="64,1024,16384,262144")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    lr = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    port = int(os.environ.get("MASTER_PORT", "29500")) + 41
    comm = mccl.Communicator(world, mccl.unique_id_from_env(os.environ.get("MASTER_ADDR", "127.0.0.1"), port), rank, transport="cuda")
    dist.init_process_group("nccl", device_id=dev)
    nxt, prv = (rank + 1) % world, (rank - 1) % world

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

    def pattern(src_rank: int, dst_rank: int, n: int) -> torch.Tensor:
        return (torch.arange(n, device=dev, dtype=torch.int32) * 7 + src_rank * 1000003 + dst_rank * 101).view(torch.uint8)

    # Ragged sizes and a misaligned buffer first (not timed): the split over channels must agree on both sides.
    ragged_ok = True
    for nbytes, shift in ((13, 0), (65536 + 5, 0), ((1 << 20) + 13, 1), ((5 << 20) + 4099, 3)):
        src = torch.arange(nbytes + shift, device=dev, dtype=torch.int64).mul_(31).add_(rank).to(torch.uint8)
        dst = torch.zeros(nbytes + shift, device=dev, dtype=torch.uint8)
        with mccl.group():
            comm.send(src[shift:], nxt)
            comm.recv(dst[shift:], prv)
        torch.cuda.synchronize()
        want = torch.arange(nbytes + shift, device=dev, dtype=torch.int64).mul_(31).add_(prv).to(torch.uint8)
        ragged_ok = ragged_ok and bool(torch.equal(dst[shift:], want[shift:])) and bool((dst[:shift] == 0).all())
    if rank == 0:
        print(json.dumps({"case": "sendrecv_ragged", "n_gpus": world, "ok": ragged_ok, "async_error": comm.async_error()}), flush=True)

    for kb in [int(x) for x in args.sizes_kb.split(",")]:
        nbytes = kb * 1024
        words = nbytes // 4
        # ---- ring
        out = pattern(rank, nxt, words)
        inn = torch.zeros(nbytes, device=dev, dtype=torch.uint8)

        def ring_mccl():
            with mccl.group():
                comm.send(out, nxt)
                comm.recv(inn, prv)

        def ring_nccl():
            for w in dist.batch_isend_irecv([dist.P2POp(dist.isend, out, nxt), dist.P2POp(dist.irecv, inn, prv)]):
                w.wait()

        ring_mccl(); torch.cuda.synchronize()
        ok_ring = bool(torch.equal(inn, pattern(prv, rank, words)))
        row = {"case": "sendrecv", "n_gpus": world, "bytes": nbytes, "ring_ok": ok_ring}
        t = timed(ring_mccl); row["ring_mccl_us"] = round(t, 1); row["ring_mccl_gbs"] = round(nbytes / t / 1e3, 1)
        t = timed(ring_nccl); row["ring_nccl_us"] = round(t, 1); row["ring_nccl_gbs"] = round(nbytes / t / 1e3, 1)
        row["ring_vs_nccl"] = round(row["ring_nccl_us"] / row["ring_mccl_us"], 3)
        # ---- all pairs (a block of nbytes / world to and from every other rank)
        if world > 2:
            blk = max(16, nbytes // world // 16 * 16)
            bw = blk // 4
            outs = [pattern(rank, p, bw) for p in range(world)]
            inns = [torch.zeros(blk, device=dev, dtype=torch.uint8) for _ in range(world)]

            def pairs_mccl():
                with mccl.group():
                    for p in range(world):
                        if p != rank:
                            comm.send(outs[p], p)
                            comm.recv(inns[p], p)

            def pairs_nccl():
                ops = []
                for p in range(world):
                    if p != rank:
                        ops += [dist.P2POp(dist.isend, outs[p], p), dist.P2POp(dist.irecv, inns[p], p)]
                for w in dist.batch_isend_irecv(ops):
                    w.wait()

            pairs_mccl(); torch.cuda.synchronize()
            row["pairs_ok"] = all(bool(torch.equal(inns[p], pattern(p, rank, bw))) for p in range(world) if p != rank)
            got = blk * (world - 1)
            t = timed(pairs_mccl); row["pairs_mccl_us"] = round(t, 1); row["pairs_mccl_gbs"] = round(got / t / 1e3, 1)
            t = timed(pairs_nccl); row["pairs_nccl_us"] = round(t, 1); row["pairs_nccl_gbs"] = round(got / t / 1e3, 1)
            row["pairs_vs_nccl"] = round(row["pairs_nccl_us"] / row["pairs_mccl_us"], 3)
        row["async_error"] = comm.async_error()
        if rank == 0:
            print(json.dumps(row), flush=True)
    comm.finalize(); comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
