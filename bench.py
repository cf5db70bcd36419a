#!/usr/bin/env python
"""Flagship benchmark: data-parallel training step of a GPT-2-medium-shaped decoder (24 layers, d_model
1024, 16 heads, FFN 4096, vocab 50257, sequence 1024, bf16, micro-batch 8 per GPU, 25 MB gradient buckets
all-reduced with a fused 1/world average while backward runs, fused AdamW step).  Weak scaling: the work
per GPU is fixed.  Prints one JSON line on rank 0.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus 8 --steps 10 --warmup 3

`--impl reference` answers for the reference library (macOS/Metal only: it cannot be installed on Linux);
`--impl nccl` runs the same step through torch DDP over NCCL, the floor this library is compared with.
"""
from __future__ import annotations

import argparse
import json
import os
import struct
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "dp_step_tokens_per_s"
REFERENCE_UNAVAILABLE = ("reference is a macOS/Metal C++ library with no Python package: pip reports 'Neither setup.py nor "
                         "pyproject.toml found', and its sources need Metal/IOKit/SO_NOSIGPIPE (CMakeLists.txt:2,30)")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="mccl", choices=["mccl", "reference", "nccl", "c10d"],
                    help="mccl: this library's DDP wrapper; nccl: torch DDP over NCCL; c10d: torch DDP over this library's "
                         "torch.distributed backend; reference: the reference library (unavailable here)")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    ap.add_argument("--model", default="gpt2-medium", choices=["gpt2-medium", "tiny"])
    ap.add_argument("--no-extras", action="store_true", help="skip the all-reduce bus-bandwidth table")
    ap.add_argument("--shard-optimizer", action="store_true",
                    help="reduce-scatter gradients, update 1/world of the parameters per rank, all-gather them (ZeRO stage 1)")
    return ap.parse_args()


def host_max(comm, value: float) -> float:
    if comm is None:
        return value
    return max(struct.unpack("d", b)[0] for b in comm.host_all_gather(struct.pack("d", value)))


def main() -> int:
    args = parse()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:          # one line per job, also under a multi-rank launch
            print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from mccl_b200.models.gpt2 import GPT2, GPT2Config
    from mccl_b200.utils.clocks import ClockSampler

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(f"bench.py: --gpus {args.gpus} needs a torchrun launch with {args.gpus} ranks", file=sys.stderr)
            return 2
        args.gpus = world
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    torch.manual_seed(1234)                      # same initial weights on every rank
    cfg = GPT2Config.medium() if args.model == "gpt2-medium" else GPT2Config.tiny()
    B, S = args.micro_batch, cfg.seq_len

    comm = None
    # The NCCL arm is what a user runs without this library: stock PyTorch loss, DDP and optimizer.
    model = GPT2(cfg, fused_loss=args.impl == "mccl").to(device=dev, dtype=torch.bfloat16)
    n_params = model.num_params()
    launches = lambda: 0
    if args.impl == "mccl":
        import mccl_b200 as mccl
        from mccl_b200.ops import loss as loss_ops
        from mccl_b200.ops import norm as norm_ops
        from mccl_b200.ops import optim
        from mccl_b200.parallel.ddp import DistributedDataParallel
        if world > 1:
            port = int(os.environ.get("MASTER_PORT", "29500")) + 23
            uid = mccl.unique_id_from_env(os.environ.get("MASTER_ADDR", "127.0.0.1"), port)
            comm = mccl.Communicator(world, uid, rank, transport="cuda")
        ddp = DistributedDataParallel(model, comm, bucket_mb=args.bucket_mb, shard_optimizer=args.shard_optimizer)
        launches = lambda: (comm.launch_count if comm is not None else 0) + optim.launches() + loss_ops.launches() + norm_ops.launches()

        def train_step(tokens):
            loss = ddp(tokens[:, :-1], tokens[:, 1:])
            loss.backward()
            ddp.step(lr=3e-4, max_grad_norm=1.0)
            return loss
    else:
        import torch.distributed as dist
        if args.impl == "c10d":
            import mccl_b200.c10d  # noqa: F401  (registers the "mccl" backend)
        if world > 1:
            dist.init_process_group("mccl" if args.impl == "c10d" else "nccl", **({} if args.impl == "c10d" else {"device_id": dev}))
        net = model
        if world > 1:
            net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], bucket_cap_mb=args.bucket_mb,
                                                            gradient_as_bucket_view=True)
        opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)

        def train_step(tokens):
            loss = net(tokens[:, :-1], tokens[:, 1:])
            loss.backward()
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0, foreach=True)
            opt.step()
            opt.zero_grad(set_to_none=False)
            return loss

    # Synthetic token ids, uniform over the vocabulary, in pinned host memory; a few distinct batches are cycled.
    g = torch.Generator().manual_seed(99 + rank)
    pool = 4
    host_tokens = torch.randint(0, cfg.vocab_size, (pool, B, S + 1), generator=g, dtype=torch.int64).pin_memory()
    dev_tokens = host_tokens.to(dev)

    def barrier():
        torch.cuda.synchronize()
        if comm is not None:
            comm.host_barrier()
        elif args.impl in ("nccl", "c10d") and world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        loss = train_step(host_tokens[i % pool].to(dev, non_blocking=True))
        loss.item()

    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    # ---- device-timed region: K steps, inputs already on the device
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = launches()
    e0.record()
    for i in range(args.steps):
        train_step(dev_tokens[i % pool])
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1) / args.steps
    my_launches = launches() - l0
    # ---- end-to-end region: every step copies its batch from pinned host memory and reads the loss back
    barrier()
    t0 = time.perf_counter()
    last = 0.0
    for i in range(args.steps):
        tokens = host_tokens[i % pool].to(dev, non_blocking=True)
        last = train_step(tokens).item()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    clocks = sampler.stop() if sampler is not None else {}

    if args.impl in ("nccl", "c10d") and world > 1:
        import torch.distributed as dist
        t = torch.tensor([dev_ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = t.tolist()
    else:
        dev_ms, e2e_ms = host_max(comm, dev_ms), host_max(comm, e2e_ms)

    # ---- exposed communication: the same step with the all-reduce switched off
    exposed_ms = None
    if args.impl == "mccl" and world > 1 and not args.shard_optimizer:
        ddp.world = 1
        for b in ddp.buckets:
            b.done_event = None
        barrier()
        e0.record()
        for i in range(args.steps):
            train_step(dev_tokens[i % pool])
        e1.record()
        barrier()
        exposed_ms = max(0.0, dev_ms - host_max(comm, e0.elapsed_time(e1) / args.steps))
        ddp.world = world

    extras = {}
    if args.impl == "mccl" and world > 1 and not args.no_extras:
        try:
            extras = allreduce_table(comm, rank, world, dev)
        except Exception as exc:  # the headline number must survive a failure here
            extras = {"error": repr(exc)[:200]}

    tokens_per_step = world * B * S
    value = tokens_per_step / (dev_ms * 1e-3)
    out = {
        "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dev_ms, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids uniform over the vocabulary; random-init weights N(0,0.02)",
        "impl": args.impl,
        "config": {"model": args.model, "params": n_params, "layers": cfg.n_layer, "d_model": cfg.d_model, "heads": cfg.n_head,
                   "ffn": cfg.d_ff, "vocab": cfg.vocab_size, "global_batch": world * B, "micro_batch": B, "seq_len": S,
                   "parallelism": f"dp{world}" + ("+zero1" if args.shard_optimizer and world > 1 else ""), "bucket_mb": args.bucket_mb, "optimizer": "adamw (fused, fp32 master), global-norm clip 1.0",
                   "l2": "working set per step (0.7 GB weights + activations) exceeds the 126 MB L2; no flush needed"},
        "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"), "reasons": clocks.get("reasons", [])},
        "e2e": {"value": round(tokens_per_step / (e2e_ms * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 3),
                "h2d_bytes_per_step": B * (S + 1) * 8, "d2h_bytes_per_step": 4},
        "gpu_launches": int(my_launches),
        "final_loss": last,
    }
    if exposed_ms is not None:
        out["exposed_comm_ms"] = round(exposed_ms, 3)
    if extras:
        out["allreduce_busbw_gbs"] = extras
    if comm is not None:
        comm.finalize()
        comm.destroy()
    if rank == 0:
        print(json.dumps(out), flush=True)
    if args.impl in ("nccl", "c10d") and world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return 0


def allreduce_table(comm, rank, world, dev):
    """Bus bandwidth of the library's all-reduce (tuner's choice, symmetric bf16 buffers, in place) next to
    NCCL's on the same GPUs: time on the device, maximum over ranks."""
    import torch
    import torch.distributed as dist
    comm.set_max_ctas(0)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    table = {}

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(); comm.host_barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return host_max(comm, e0.elapsed_time(e1) / iters)

    for mb in (64, 256, 1024):
        n = mb * (1 << 20) // 2
        buf = comm.empty(n, torch.bfloat16)
        buf.normal_()
        ref = torch.empty(n, device=dev, dtype=torch.bfloat16).normal_()
        ms_m = timed(lambda: comm.all_reduce(buf, op="sum"), 10)
        algo = comm.last_algo
        ms_n = timed(lambda: dist.all_reduce(ref), 10)
        k = 2 * (world - 1) / world
        table[f"{mb}MB"] = {"mccl": round(n * 2 / ms_m / 1e6 * k, 1), "nccl": round(n * 2 / ms_n / 1e6 * k, 1), "algo": algo}
        comm.free_raw(buf.data_ptr())
        del buf, ref
    dist.destroy_process_group()
    return table


if __name__ == "__main__":
    sys.exit(main())
