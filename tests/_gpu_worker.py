"""One rank of a multi-GPU test of the cuda transport (one process per GPU).  Scenario in argv[1]."""
from __future__ import annotations

import json
import os
import sys
import time

import torch

import mccl_b200 as mccl
from mccl_b200 import _lib as L

RANK = int(os.environ["MCCL_TEST_RANK"])
WORLD = int(os.environ["MCCL_TEST_WORLD"])
PORT = int(os.environ["MCCL_TEST_PORT"])
ARGS = json.loads(os.environ.get("MCCL_TEST_ARGS", "{}"))
torch.cuda.set_device(RANK)
DEV = torch.device("cuda", RANK)


def make_comm():
    return mccl.Communicator(WORLD, mccl.unique_id_from_env("127.0.0.1", PORT), RANK, transport="cuda")


def gen(r, n, dtype):
    g = torch.Generator(device="cuda").manual_seed(1000 + r)
    if not dtype.is_floating_point:
        return torch.randint(-1000, 1000, (n,), generator=g, device="cuda", dtype=torch.int64).to(dtype)
    return (torch.rand(n, generator=g, device="cuda") * 2 - 1).to(dtype)


def oracle(n, dtype, op, seed_shift=0):
    """fp64 (or exact integer) restatement of the reduction over every rank's input."""
    xs = [gen(r + seed_shift, n, dtype) for r in range(WORLD)]
    st = torch.stack([x.double() for x in xs]) if dtype.is_floating_point else torch.stack([x.long() for x in xs])
    if op in ("sum", "avg"):
        o = st.sum(0)
        if op == "avg":
            o = o / WORLD if dtype.is_floating_point else torch.div(o.to(dtype), WORLD, rounding_mode="trunc")
    elif op == "prod":
        o = st.prod(0)
    elif op == "max":
        o = st.max(0).values
    else:
        o = st.min(0).values
    return o


def check(what, got, ref, dtype):
    if dtype.is_floating_point:
        tol = {torch.float32: 1e-5, torch.float64: 1e-12, torch.float16: 4e-3, torch.bfloat16: 3e-2}[dtype]
        err = ((got.double() - ref.double()).abs() / (ref.double().abs() + 1.0)).max().item()
        assert err <= tol, (what, err)
    else:
        assert torch.equal(got, ref.to(got.dtype)), what          # integers are bit exact


def canary_ok(comm):
    return comm.async_error() == L.SUCCESS and comm.guards_intact()


def matrix():
    comm = make_comm()
    quick = ARGS.get("quick", False)
    sizes = [4, 1024 + 3, (1 << 20) + 8] if quick else [1, 4, 1027, 65536, (1 << 20) + 8, 6 << 20]
    algos = ["oneshot", "twoshot", "ring", "tree"] + (["nvls"] if comm.nvls else [])
    dtypes = [torch.float32, torch.bfloat16, torch.float16, torch.int32] + ([] if quick else [torch.int64, torch.float64, torch.uint8])
    for dtype in dtypes:
        for n in sizes:
            for sym in (False, True):
                for algo in algos:
                    ops = ("sum", "avg") if algo == "nvls" else (("sum", "avg", "max", "min", "prod") if n <= 1027 else ("sum", "avg"))
                    for op in ops:
                        if dtype == torch.uint8 and op in ("avg", "prod"):
                            continue
                        x = gen(RANK, n, dtype)
                        if op == "prod":          # keep products representable: factors in {-1, 1} or near 1
                            x = torch.sign(x) + (x == 0).to(dtype) if not dtype.is_floating_point else (1 + x / 64).to(dtype)
                        buf = comm.empty(n, dtype) if sym else torch.empty(n, device=DEV, dtype=dtype)
                        buf.copy_(x)
                        with mccl.forced_algo(algo):
                            comm.all_reduce(buf, op=op)
                        torch.cuda.synchronize()
                        assert canary_ok(comm), ("async error", dtype, n, sym, algo, op)
                        if op == "prod":
                            xs = []
                            for r in range(WORLD):
                                y = gen(r, n, dtype)
                                xs.append((torch.sign(y) + (y == 0).to(dtype)).long() if not dtype.is_floating_point else (1 + y / 64).to(dtype).double())
                            ref = torch.stack(xs).prod(0)
                        else:
                            ref = oracle(n, dtype, op)
                        if dtype == torch.uint8:
                            ref = ref % 256 if op == "sum" else ref
                        check(("allreduce", dtype, n, sym, algo, comm.last_algo, op), buf, ref, dtype)
                        if sym:
                            comm.free_raw(buf.data_ptr())
    # out of place, sources untouched
    x = gen(RANK, 70001, torch.float32); keep = x.clone(); y = torch.empty_like(x)
    comm.all_reduce(x, y, op="sum"); torch.cuda.synchronize()
    assert torch.equal(x, keep)
    check("out-of-place", y, oracle(70001, torch.float32, "sum"), torch.float32)
    comm.finalize(); comm.destroy()


def collectives():
    comm = make_comm()
    for dtype in (torch.float32, torch.bfloat16, torch.int32):
        for n in (5, 1024 + 3, 1 << 18):
            for sym in (False, True):
                mk = (lambda m: comm.empty(m, dtype)) if sym else (lambda m: torch.empty(m, device=DEV, dtype=dtype))
                for algo in ["auto", "oneshot", "twoshot"] + (["nvls"] if comm.nvls else []):
                    with mccl.forced_algo(algo):
                        x = gen(RANK, n, dtype)
                        s = mk(n); s.copy_(x); g = mk(n * WORLD)
                        comm.all_gather(s, g); torch.cuda.synchronize()
                        assert torch.equal(g, torch.cat([gen(r, n, dtype) for r in range(WORLD)])), ("allgather", dtype, n, sym, algo)
                        g2 = mk(n * WORLD); g2[RANK * n:(RANK + 1) * n].copy_(x)
                        comm.all_gather(g2[RANK * n:(RANK + 1) * n], g2); torch.cuda.synchronize()        # in place
                        assert torch.equal(g2, g), ("allgather in place", dtype, n, sym, algo)
                        s2 = mk(n * WORLD); s2.copy_(gen(RANK + 50, n * WORLD, dtype)); o2 = mk(n)
                        comm.reduce_scatter(s2, o2, op="sum"); torch.cuda.synchronize()
                        check(("reducescatter", dtype, n, sym, algo), o2, oracle(n * WORLD, dtype, "sum", 50)[RANK * n:(RANK + 1) * n], dtype)
                        for root in {0, WORLD - 1}:
                            b = mk(n); b.zero_()
                            if RANK == root:
                                b.copy_(x)
                            comm.broadcast(b if RANK == root else None, b, root=root); torch.cuda.synchronize()
                            assert torch.equal(b, gen(root, n, dtype)), ("broadcast", dtype, n, sym, algo, root)
                            s3 = mk(n); s3.copy_(x); o3 = mk(n)
                            comm.reduce(s3, o3, op="avg" if dtype.is_floating_point else "sum", root=root); torch.cuda.synchronize()
                            if RANK == root:
                                check(("reduce", dtype, n, sym, algo, root), o3, oracle(n, dtype, "avg" if dtype.is_floating_point else "sum"), dtype)
                        for t in (s, g, g2, s2, o2):
                            if sym:
                                comm.free_raw(t.data_ptr())
                blk = max(n // WORLD, 1)
                s4 = mk(blk * WORLD); s4.copy_(gen(RANK, blk * WORLD, dtype)); o4 = mk(blk * WORLD)
                comm.all_to_all(s4, o4); torch.cuda.synchronize()
                ref = torch.cat([gen(p, blk * WORLD, dtype)[RANK * blk:(RANK + 1) * blk] for p in range(WORLD)])
                assert torch.equal(o4, ref), ("alltoall", dtype, n, sym)
        assert canary_ok(comm)
    # Send/Recv ring inside a group (both directions at once), odd size
    x = gen(RANK, 3_000_001, torch.float32); y = torch.empty_like(x); z = torch.empty_like(x)
    with mccl.group():
        comm.send(x, (RANK + 1) % WORLD); comm.recv(y, (RANK - 1) % WORLD)
        comm.send(x, (RANK - 1) % WORLD); comm.recv(z, (RANK + 1) % WORLD)
    torch.cuda.synchronize()
    assert torch.equal(y, gen((RANK - 1) % WORLD, 3_000_001, torch.float32))
    assert torch.equal(z, gen((RANK + 1) % WORLD, 3_000_001, torch.float32))
    if RANK == 0:
        seen = set()
        for _ in range(WORLD - 1):
            buf = torch.empty(256, device=DEV)
            src = comm.recv_any(buf); torch.cuda.synchronize()
            assert torch.all(buf == float(src)); seen.add(src)
        assert seen == set(range(1, WORLD))
    else:
        comm.send(torch.full((256,), float(RANK), device=DEV), 0)
    torch.cuda.synchronize()
    comm.finalize(); comm.destroy()


def split_and_ddp():
    from mccl_b200.models.gpt2 import GPT2, GPT2Config
    from mccl_b200.parallel.ddp import DistributedDataParallel
    comm = make_comm()
    sub = comm.split(RANK % 2, RANK)
    members = [r for r in range(WORLD) if r % 2 == RANK % 2]
    y = torch.full((1000,), RANK + 1.0, device=DEV)
    sub.all_reduce(y); torch.cuda.synchronize()
    assert torch.all(y == sum(r + 1.0 for r in members))
    sub.finalize(); sub.destroy()
    torch.manual_seed(0)
    cfg = GPT2Config.tiny()
    model = GPT2(cfg).to(device=DEV, dtype=torch.bfloat16)
    ddp = DistributedDataParallel(model, comm, bucket_mb=0.25)
    g = torch.Generator().manual_seed(7 + RANK)
    tokens = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len + 1), generator=g).to(DEV)
    losses = []
    for _ in range(5):
        loss = ddp(tokens[:, :-1], tokens[:, 1:]); loss.backward(); ddp.step(lr=3e-3)
        losses.append(loss.item())
    assert losses[-1] < losses[0], losses
    # replicas stay bit-identical: same averaged gradients, same optimizer arithmetic
    flat = torch.cat([b.param.float() for b in ddp.buckets])
    gathered = torch.empty(flat.numel() * WORLD, device=DEV)
    comm.all_gather(flat, gathered); torch.cuda.synchronize()
    for r in range(WORLD):
        assert torch.equal(gathered[r * flat.numel():(r + 1) * flat.numel()], flat), f"replica {r} diverged"
    comm.finalize(); comm.destroy()


def ddp_graphed():
    """The whole step recorded in a CUDA graph (bucket all-reduces on their side stream included) follows the same
    trajectory as the step issued kernel by kernel, and the replicas stay bit-identical."""
    from mccl_b200.models.gpt2 import GPT2, GPT2Config
    from mccl_b200.parallel.ddp import DistributedDataParallel
    comm = make_comm()
    cfg = GPT2Config.tiny()
    g = torch.Generator().manual_seed(7 + RANK)
    batches = torch.randint(0, cfg.vocab_size, (3, 4, cfg.seq_len + 1), generator=g).to(DEV)

    def build():
        torch.manual_seed(0)
        return DistributedDataParallel(GPT2(cfg).to(device=DEV, dtype=torch.bfloat16), comm, bucket_mb=0.25)

    eager = build()
    ref = []
    for i in range(7):
        t = batches[i % 3]
        loss = eager(t[:, :-1], t[:, 1:]); loss.backward(); eager.step(lr=3e-3, max_grad_norm=1.0)
        ref.append(loss.item())
    ddp = build()
    t = batches[0]
    step = ddp.graphed_step((t[:, :-1], t[:, 1:]), lr=3e-3, max_grad_norm=1.0, warmup=1)     # the warm-up is step 0
    got = [ref[0]]
    for i in range(1, 7):
        t = batches[i % 3]
        got.append(step(t[:, :-1], t[:, 1:]).item())
    assert step.launches_per_step > 0 and ddp.step_count == 7
    for a, b in zip(ref, got):
        assert abs(a - b) < 2e-2 * max(1.0, abs(a)), (ref, got)
    assert got[-1] < got[1], got
    torch.cuda.synchronize()
    assert canary_ok(comm)
    flat = torch.cat([b.param.float() for b in ddp.buckets])
    gathered = torch.empty(flat.numel() * WORLD, device=DEV)
    comm.all_gather(flat, gathered); torch.cuda.synchronize()
    for r in range(WORLD):
        assert torch.equal(gathered[r * flat.numel():(r + 1) * flat.numel()], flat), f"replica {r} diverged"
    comm.finalize(); comm.destroy()


def ddp_sharded():
    """Sharded optimizer on GPUs: same losses as the replicated optimizer step for step (same averaged gradients,
    same arithmetic per element, clipping by the same global norm), replicas bit-identical, state 1/world."""
    from mccl_b200.models.gpt2 import GPT2, GPT2Config
    from mccl_b200.parallel.ddp import DistributedDataParallel
    comm = make_comm()
    cfg = GPT2Config.tiny()
    g = torch.Generator().manual_seed(7 + RANK)
    tokens = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len + 1), generator=g).to(DEV)
    runs = []
    for shard in (False, True):
        torch.manual_seed(0)
        model = GPT2(cfg).to(device=DEV, dtype=torch.bfloat16)
        ddp = DistributedDataParallel(model, comm, bucket_mb=0.25, shard_optimizer=shard)
        losses = []
        for _ in range(5):
            loss = ddp(tokens[:, :-1], tokens[:, 1:]); loss.backward(); ddp.step(lr=3e-3, max_grad_norm=1.0)
            losses.append(loss.item())
        torch.cuda.synchronize()
        flat = torch.cat([b.param[:sum((p.numel() + 7) // 8 * 8 for p in b.params)].float() for b in ddp.buckets])
        runs.append((losses, flat, ddp))
    (l0, p0, d0), (l1, p1, d1) = runs
    assert l1[-1] < l1[0], l1
    assert max(abs(a - b) for a, b in zip(l0, l1)) < 2e-2, (l0, l1)
    assert (p0 - p1).abs().max().item() < 2e-2, (p0 - p1).abs().max().item()     # a few bf16 steps after 5 updates
    assert all(b.master.numel() * WORLD == b.numel for b in d1.buckets)
    gathered = torch.empty(p1.numel() * WORLD, device=DEV)
    comm.all_gather(p1.contiguous(), gathered); torch.cuda.synchronize()
    for r in range(WORLD):
        assert torch.equal(gathered[r * p1.numel():(r + 1) * p1.numel()], p1), f"replica {r} diverged"
    assert canary_ok(comm)
    comm.finalize(); comm.destroy()


def c10d_backend_gpu():
    """The "mccl" torch.distributed backend on cuda tensors: plain c10d calls, then torch's DistributedDataParallel
    (bucket hooks use the work's future) against single-process training on the whole batch."""
    import torch.distributed as dist
    import mccl_b200.c10d  # noqa: F401
    dist.init_process_group("mccl", rank=RANK, world_size=WORLD, init_method="file://" + ARGS["rendezvous"])
    n = WORLD
    t = torch.full((1 << 20,), RANK + 1.0, device=DEV)
    dist.all_reduce(t)
    assert torch.all(t == n * (n + 1) / 2)
    w = dist.all_reduce(t, op=dist.ReduceOp.AVG, async_op=True)
    w.wait()
    assert torch.all(t == n * (n + 1) / 2)
    b = torch.arange(1000, device=DEV, dtype=torch.int64) * (1 if RANK == n - 1 else 0)
    dist.broadcast(b, src=n - 1)
    assert torch.equal(b, torch.arange(1000, device=DEV, dtype=torch.int64))
    out = torch.empty(4096 * n, device=DEV, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(out, torch.full((4096,), float(RANK), device=DEV, dtype=torch.bfloat16))
    assert torch.equal(out.float(), torch.arange(n, device=DEV, dtype=torch.float32).repeat_interleave(4096))
    rs = torch.empty(512, device=DEV)
    dist.reduce_scatter_tensor(rs, torch.arange(512 * n, device=DEV, dtype=torch.float32))
    assert torch.equal(rs, n * torch.arange(512 * RANK, 512 * RANK + 512, device=DEV, dtype=torch.float32))
    dist.barrier()
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.Tanh(), torch.nn.Linear(256, 8)).to(DEV)
    ref = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.Tanh(), torch.nn.Linear(256, 8)).to(DEV)
    ref.load_state_dict(net.state_dict())
    ddp = torch.nn.parallel.DistributedDataParallel(net, device_ids=[RANK], bucket_cap_mb=0.01)
    g = torch.Generator().manual_seed(3)
    x, y = torch.randn(8 * n, 64, generator=g).to(DEV), torch.randn(8 * n, 8, generator=g).to(DEV)
    o1, o2 = torch.optim.SGD(ddp.parameters(), lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    for _ in range(3):
        o1.zero_grad(); torch.nn.functional.mse_loss(ddp(x[8 * RANK:8 * RANK + 8]), y[8 * RANK:8 * RANK + 8]).backward(); o1.step()
        o2.zero_grad(); torch.nn.functional.mse_loss(ref(x), y).backward(); o2.step()
    torch.cuda.synchronize()
    for p1, p2 in zip(net.parameters(), ref.parameters()):
        assert torch.allclose(p1, p2, atol=1e-5, rtol=1e-4), (p1 - p2).abs().max().item()
    # torch FSDP2 on cuda: its own all-gather / reduce-scatter streams wait on this backend's work objects
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard
    mesh = init_device_mesh("cuda", (n,))
    torch.manual_seed(1)
    fs = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.Tanh(), torch.nn.Linear(256, 8)).to(DEV)
    ref = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.Tanh(), torch.nn.Linear(256, 8)).to(DEV)
    ref.load_state_dict(fs.state_dict())
    for layer in (fs[0], fs[2]):
        fully_shard(layer, mesh=mesh)
    fully_shard(fs, mesh=mesh)
    o1, o2 = torch.optim.SGD(fs.parameters(), lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    for _ in range(3):
        o1.zero_grad(); torch.nn.functional.mse_loss(fs(x[8 * RANK:8 * RANK + 8]), y[8 * RANK:8 * RANK + 8]).backward(); o1.step()
        o2.zero_grad(); torch.nn.functional.mse_loss(ref(x), y).backward(); o2.step()
    torch.cuda.synchronize()
    for p1, p2 in zip(fs.parameters(), ref.parameters()):
        assert torch.allclose(p1.full_tensor(), p2, atol=1e-5, rtol=1e-4), (p1.full_tensor() - p2).abs().max().item()
    dist.destroy_process_group()


def parallel_layers_gpu():
    """The model-parallel layers and the pipeline schedule on cuda tensors (fp32, collectives through the kernels)."""
    from _parallel_cases import fsdp_case, layers_case, llama_case, pipeline_case
    comm = make_comm()
    fsdp_case(comm, RANK, WORLD, DEV, atol=2e-4)
    layers_case(comm, RANK, WORLD, DEV, atol=2e-4)
    pipeline_case(comm, RANK, WORLD, DEV, atol=1e-5)
    llama_case(comm, RANK, WORLD, DEV, atol=2e-4)
    assert canary_ok(comm)
    comm.finalize(); comm.destroy()


def moe_fused():
    """The fused dispatch / combine kernels against the pack + all-to-all + unpack form of the same layer: outputs and
    the gradients of the tokens, the router and the experts, fp32 and bf16, with dropped tokens."""
    from mccl_b200.parallel import layers as PL
    comm = make_comm()
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
        hid, ffn, e_loc, cap = 64, 128, 2, 3
        T = e_loc * WORLD * cap + 5
        torch.manual_seed(0)
        a = PL.ExpertParallelMoE(comm, hid, ffn, e_loc, cap, device=DEV, dtype=dtype, fused=False)
        b = PL.ExpertParallelMoE(comm, hid, ffn, e_loc, cap, device=DEV, dtype=dtype, fused=True)
        b.load_state_dict(a.state_dict())
        g = torch.Generator(device="cuda").manual_seed(50 + RANK)
        x = torch.randn(T, hid, device=DEV, generator=g).to(dtype)
        tgt = torch.randn(T, hid, device=DEV, generator=g).to(dtype)
        outs = []
        for m in (a, b):
            xi = x.clone().requires_grad_(True)
            y = m(xi)
            (y.float() * tgt.float()).sum().backward()
            outs.append((y.detach().float(), xi.grad.float(), m.router.weight.grad.float(), m.w_in.grad.float(), m.w_out.grad.float()))
        torch.cuda.synchronize()
        assert (outs[0][0].abs().sum(-1) == 0).any(), "nothing was dropped"
        for name, u, v in zip(("y", "dx", "d router", "d w_in", "d w_out"), outs[0], outs[1]):
            err = ((u - v).abs().max() / (u.abs().max() + 1e-6)).item()
            assert err < tol, (dtype, name, err)
    assert canary_ok(comm)
    comm.finalize(); comm.destroy()


def tp_mlp_trainable():
    """FusedTensorParallelMLP (fused forward kernels, collective backward) against the unfused sequence-parallel MLP
    with the same weights: output and the gradients of the input and both weight shards."""
    from mccl_b200.parallel.layers import TensorParallelMLP
    from mccl_b200.parallel.tp import FusedTensorParallelMLP
    comm = make_comm()
    tokens, hidden, ffn = 128 * WORLD * 2, 512, 256 * WORLD
    torch.manual_seed(5 + RANK)
    fused = FusedTensorParallelMLP(comm, tokens, hidden, ffn, device=DEV)
    plain = TensorParallelMLP(comm, hidden, ffn, bias=False, sequence_parallel=True, device=DEV, dtype=torch.bfloat16)
    with torch.no_grad():
        plain.up.weight.copy_(fused.w_up); plain.down.weight.copy_(fused.w_down)
    g = torch.Generator(device="cuda").manual_seed(70 + RANK)
    x = torch.randn(tokens // WORLD, hidden, device=DEV, generator=g).to(torch.bfloat16)
    tgt = torch.randn(tokens // WORLD, hidden, device=DEV, generator=g).to(torch.bfloat16)
    res = []
    for m, wu, wd in ((plain, plain.up.weight, plain.down.weight), (fused, fused.w_up, fused.w_down)):
        for it in range(2):                                     # the second pass reuses flags and buffers
            wu.grad = wd.grad = None
            xi = x.clone().requires_grad_(True)
            y = m(xi)
            (y.float() * tgt.float()).sum().backward()
        res.append((y.detach().float(), xi.grad.float(), wu.grad.float(), wd.grad.float()))
    torch.cuda.synchronize()
    from mccl_b200.ops import gemm as G
    assert G.last_error() == 0 and comm.async_error() == L.SUCCESS
    for name, u, v in zip(("y", "dx", "d w_up", "d w_down"), res[0], res[1]):
        err = ((u - v).abs().max() / (u.abs().max() + 1e-6)).item()
        assert err < 3e-2, (name, err)
    comm.finalize(); comm.destroy()


def rooted_and_ragged_gpu():
    """mcclGather, mcclScatter and mcclAllToAllv on cuda tensors (the batched Send / Recv kernel underneath)."""
    comm = make_comm()
    n, r = WORLD, RANK
    for root in (0, n - 1):
        out = torch.zeros(5000 * n, device=DEV) if r == root else None
        comm.gather(torch.full((5000,), float(r), device=DEV), out, root=root); torch.cuda.synchronize()
        if r == root:
            assert torch.equal(out, torch.arange(n, device=DEV, dtype=torch.float32).repeat_interleave(5000))
        piece = torch.zeros(3001, device=DEV, dtype=torch.int64)
        comm.scatter(torch.arange(3001 * n, device=DEV, dtype=torch.int64) if r == root else None, piece, root=root); torch.cuda.synchronize()
        assert torch.equal(piece, torch.arange(3001 * r, 3001 * r + 3001, device=DEV, dtype=torch.int64))
    k = 70_001                                                    # odd segment sizes, several FIFO chunks
    send = torch.cat([torch.full(((j + 1) * k,), 100.0 * r + j, device=DEV) for j in range(n)])
    recv = torch.zeros(n * (r + 1) * k, device=DEV)
    comm.all_to_all_v(send, [(j + 1) * k for j in range(n)], recv, [(r + 1) * k] * n); torch.cuda.synchronize()
    assert torch.equal(recv, torch.cat([torch.full(((r + 1) * k,), 100.0 * s + r, device=DEV) for s in range(n)]))
    assert canary_ok(comm)
    comm.finalize(); comm.destroy()


def device_timeout():
    """Rank 1 sits out one collective (between steps, nothing of its own in flight).  The others' kernels
    give up after the device time budget, record why in the status word and return; the host reads it."""
    comm = make_comm()
    x = torch.ones(1 << 16, device=DEV)
    comm.all_reduce(x); torch.cuda.synchronize()
    assert comm.async_error() == L.SUCCESS
    comm.host_barrier()
    if RANK == 1:
        time.sleep(4.0)                     # takes no part in the next collective
    else:
        t0 = time.time()
        comm.all_reduce(x); torch.cuda.synchronize()          # returns: the wait is bounded
        assert time.time() - t0 < 10
        assert comm.async_error() == L.REMOTE_ERROR
        try:
            comm.all_reduce(x)
            raise SystemExit("a poisoned communicator accepted more work")
        except mccl.MCCLError as e:
            assert e.code == L.REMOTE_ERROR
        y = torch.ones(8, device=DEV) * 3              # the CUDA context is intact
        assert y.sum().item() == 24
    comm.abort(); comm.destroy()


def forced_ring_tree():
    """Ring and tree forms of all-gather, reduce-scatter, broadcast and reduce (partial phases of the ring and tree
    kernels plus a scatter before or a collect after), symmetric and staged, sizes that do and do not meet the
    16-byte rule (the latter fall back)."""
    comm = make_comm()
    ftol = lambda dtype: 3e-2 * WORLD if dtype == torch.bfloat16 else 1e-5
    cases = [(dtype, n, sym) for dtype in (torch.float32, torch.bfloat16) for n in (8, 1000, 1027, 1 << 18) for sym in (False, True)]
    for dtype, n, sym in cases:
        mk = (lambda m: comm.empty(m, dtype)) if sym else (lambda m: torch.empty(m, device=DEV, dtype=dtype))
        x = gen(RANK, n, dtype)
        for algo in ("ring", "tree"):
            # by default the native pairs (ring: all-gather / reduce-scatter, tree: broadcast / reduce); "composed"
            # adds the forms built from a partial phase plus a scatter or a collect
            sharded = algo == "ring" or ARGS.get("composed", False)
            rooted = algo == "tree" or ARGS.get("composed", False)
            with mccl.forced_algo(algo):
                if sharded:
                    s = mk(n); s.copy_(x); g = mk(n * WORLD)
                    comm.all_gather(s, g); torch.cuda.synchronize()
                    assert torch.equal(g, torch.cat([gen(r, n, dtype) for r in range(WORLD)])), (algo, "allgather", dtype, n, sym, comm.last_algo)
                    s2 = mk(n * WORLD); s2.copy_(gen(RANK + 50, n * WORLD, dtype)); keep = s2.clone(); o2 = mk(n)
                    comm.reduce_scatter(s2, o2, op="avg"); torch.cuda.synchronize()
                    assert torch.equal(s2, keep), "reduce-scatter must not modify its input"
                    ref = oracle(n * WORLD, dtype, "avg", 50)[RANK * n:(RANK + 1) * n]
                    err = ((o2.double() - ref).abs() / (ref.abs() + 1.0)).max().item()
                    assert err < ftol(dtype), (algo, "reducescatter", dtype, n, sym, err)
                if rooted:
                    for root in {0, WORLD - 1}:
                        b = mk(n); b.zero_()
                        if RANK == root:
                            b.copy_(x)
                        comm.broadcast(b if RANK == root else None, b, root=root); torch.cuda.synchronize()
                        assert torch.equal(b, gen(root, n, dtype)), (algo, "broadcast", dtype, n, sym, root, comm.last_algo)
                        s3 = mk(n); s3.copy_(x); o3 = mk(n)
                        comm.reduce(s3, o3, op="sum", root=root); torch.cuda.synchronize()
                        assert torch.equal(s3, x), "reduce must not modify its input"
                        if RANK == root:
                            ref = oracle(n, dtype, "sum")
                            err = ((o3.double() - ref).abs() / (ref.abs() + 1.0)).max().item()
                            assert err < ftol(dtype), (algo, "reduce", dtype, n, sym, root, err)
        assert canary_ok(comm)
    comm.finalize(); comm.destroy()


def register_user_buffer():
    """mcclCommRegister: a tensor from torch's allocator becomes peer-visible (CUDA IPC) and is reduced in place."""
    comm = make_comm()
    n = (1 << 20) + 4
    x = torch.empty(n, device=DEV, dtype=torch.float32)
    peer = (RANK + 1) % WORLD
    assert comm.peer_pointer(x, peer) == 0
    before = comm.launch_count
    h = comm.register(x)
    assert comm.peer_pointer(x, peer) != 0 and comm.peer_pointer(x, RANK) == x.data_ptr()
    x.copy_(gen(RANK, n, torch.float32))
    with mccl.forced_algo("twoshot"):
        comm.all_reduce(x, op="sum")
    torch.cuda.synchronize()
    check("registered all-reduce", x, oracle(n, torch.float32, "sum"), torch.float32)
    assert comm.launch_count - before == 1, "a registered buffer needs no staging copies"
    g = torch.empty(n * WORLD, device=DEV, dtype=torch.float32)
    comm.all_gather(x, g); torch.cuda.synchronize()          # registered source, plain destination
    assert torch.equal(g[RANK * n:(RANK + 1) * n], x)
    comm.deregister(h)
    assert comm.peer_pointer(x, peer) == 0
    y = gen(RANK, 1000, torch.float32)
    comm.all_reduce(y); torch.cuda.synchronize()             # staging path still fine afterwards
    check("after deregister", y, oracle(1000, torch.float32, "sum"), torch.float32)
    comm.finalize(); comm.destroy()


def large_root_collectives():
    """Broadcast and reduce of a message large enough for the many-CTA root-only NVLS path, plus a 1 GB
    all-reduce (round-robin work tiles), against the oracle."""
    comm = make_comm()
    n = 12 << 20                                   # 48 MB of fp32
    for root in (0, WORLD - 1):
        b = comm.empty(n, torch.float32); b.zero_()
        if RANK == root:
            b.copy_(gen(root, n, torch.float32))
        comm.broadcast(b if RANK == root else None, b, root=root); torch.cuda.synchronize()
        assert torch.equal(b, gen(root, n, torch.float32)), ("broadcast", root, comm.last_algo)
        s = comm.empty(n, torch.float32); s.copy_(gen(RANK, n, torch.float32))
        o = comm.empty(n, torch.float32)
        comm.reduce(s, o, op="sum", root=root); torch.cuda.synchronize()
        if RANK == root:
            check(("reduce", root, comm.last_algo), o, oracle(n, torch.float32, "sum"), torch.float32)
        for t in (b, s, o):
            comm.free_raw(t.data_ptr())
    n = 1 << 29                                    # 1 GB of bf16
    x = comm.empty(n, torch.bfloat16)
    x.copy_(gen(RANK, n, torch.bfloat16))
    comm.all_reduce(x, op="avg"); torch.cuda.synchronize()
    ref = oracle(n, torch.bfloat16, "avg")
    check(("allreduce 1GB", comm.last_algo), x, ref, torch.bfloat16)
    assert canary_ok(comm)
    comm.finalize(); comm.destroy()


def rooted_spread():
    """MCCL_NVLS_SPREAD=1: broadcast and reduce with one shard per rank.  In place, out of place inside one
    allocation (the root publishes the offset), and with a destination the peers cannot reach (the root then
    reduces alone); every root; sizes around the shard boundaries."""
    comm = make_comm()
    for dtype in (torch.float32, torch.bfloat16):
        for n in (WORLD * 8, 4096 + 8, (3 << 20) + 64):
            for root in range(WORLD):
                b = comm.empty(n, dtype); b.zero_()
                src = gen(root, n, dtype)
                comm.broadcast(src if RANK == root else None, b, root=root); torch.cuda.synchronize()   # out of place on the root
                assert torch.equal(b, src), ("broadcast", dtype, n, root, comm.last_algo)
                two = comm.empty(2 * n, dtype)                  # source and destination halves of one allocation
                s, o = two[:n], two[n:]
                s.copy_(gen(RANK, n, dtype)); o.zero_()
                ref = oracle(n, dtype, "sum")
                comm.reduce(s, o, op="sum", root=root); torch.cuda.synchronize()
                if RANK == root:
                    check(("reduce same allocation", dtype, n, root, comm.last_algo), o, ref, dtype)
                assert torch.equal(s, gen(RANK, n, dtype)), "reduce changed its source"
                other = torch.zeros(n, device=DEV, dtype=dtype)   # not symmetric: the root works alone
                comm.reduce(s, other, op="sum", root=root); torch.cuda.synchronize()
                if RANK == root:
                    check(("reduce alone", dtype, n, root), other, ref, dtype)
                comm.reduce(s, s, op="avg", root=root); torch.cuda.synchronize()   # in place
                if RANK == root:
                    check(("reduce in place", dtype, n, root), s, oracle(n, dtype, "avg"), dtype)
                for t in (b, two):
                    comm.free_raw(t.data_ptr())
    assert canary_ok(comm)
    comm.finalize(); comm.destroy()


def graph_capture():
    """Collectives captured into a CUDA graph and replayed: every counter the kernels synchronise through lives in
    device memory, so a replay is a new, valid call.  Small (one-shot), medium and large (NVLS / two-shot) sizes."""
    comm = make_comm()
    side = torch.cuda.Stream()
    for n in (1 << 10, 1 << 18, 1 << 23):
        x = comm.empty(n, torch.float32)
        x.fill_(float(RANK + 1))
        y = comm.empty(n * WORLD, torch.float32)
        torch.cuda.synchronize(); comm.host_barrier()
        with torch.cuda.stream(side):
            comm.all_reduce(x, op="sum")                 # warm-up outside the capture
        torch.cuda.synchronize(); comm.host_barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            comm.all_reduce(x, op="sum")
            comm.all_gather(x, y)
        total = WORLD * (WORLD + 1) // 2                  # after the warm-up every rank holds `total`
        for replay in range(1, 4):
            g.replay(); torch.cuda.synchronize()
            want = float(total * WORLD ** replay)
            assert torch.all(x == want), ("graph all_reduce", n, replay, x[:4].tolist(), want)
            assert torch.all(y == want), ("graph all_gather", n, replay)
        assert canary_ok(comm)
        del g
        for t in (x, y):
            comm.free_raw(t.data_ptr())
    comm.finalize(); comm.destroy()


def calibrate_and_trace():
    """MCCL_CALIBRATE=1 measures pair bandwidth and empty-collective latency at init and feeds the tuner;
    MCCL_TRACE writes a Chrome trace with a device track."""
    import json as js
    import xml.etree.ElementTree as ET
    comm = make_comm()
    root = ET.fromstring(comm.topo_xml())
    links = [l for g in root.findall("gpu") for l in g.findall("link")]
    assert links and all(float(l.get("measured", "0")) > 10.0 for l in links), [l.attrib for l in links][:2]
    assert all(0.0 < float(l.get("latency_us", "0")) < 1000.0 for l in links)
    x = torch.ones(1 << 20, device=DEV)
    comm.all_reduce(x); comm.all_reduce(x, op="avg"); torch.cuda.synchronize()
    assert torch.all(x == WORLD)
    comm.finalize(); comm.destroy()
    data = js.load(open(os.environ["MCCL_TRACE"] + f".{RANK}.json"))
    dev_events = [e for e in data["traceEvents"] if e["cat"] == "device"]
    assert len(dev_events) == 2 and all(e["dur"] > 0 for e in dev_events), data


def tp_ffn():
    """Fused all-gather->GEMM->SiLU and GEMM->reduce-scatter against an fp32 PyTorch restatement."""
    from mccl_b200.parallel.tp import TensorParallelFFN
    comm = make_comm()
    tokens, hidden, ffn = ARGS.get("tokens", 128 * WORLD * 2), ARGS.get("hidden", 512), ARGS.get("ffn", 256 * WORLD)
    def mk(seed, shape, scale):
        g = torch.Generator(device="cuda").manual_seed(seed)
        return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)
    xs = [mk(10 + r, (tokens // WORLD, hidden), 1.0) for r in range(WORLD)]
    wus = [mk(100 + r, (ffn // WORLD, hidden), 0.05) for r in range(WORLD)]
    wds = [mk(200 + r, (hidden, ffn // WORLD), 0.05) for r in range(WORLD)]
    layer = TensorParallelFFN(comm, tokens, hidden, ffn, wus[RANK].contiguous(), wds[RANK].contiguous())
    ref = layer.reference(xs, wus, wds)
    from mccl_b200.ops import gemm as G
    for it in range(3):                       # repeated calls reuse flags and staging
        out = layer.forward(xs[RANK])
        torch.cuda.synchronize()
        assert G.last_error() == 0 and comm.async_error() == L.SUCCESS, (G.last_error(), comm.async_error())
        x_all = torch.cat(xs)
        assert torch.equal(layer.x_full, x_all), "gathered activations differ"
        href = torch.nn.functional.silu(x_all.float() @ wus[RANK].float().t())
        eh = ((layer.h.float() - href).abs() / (href.abs() + 1.0)).max().item()
        assert eh < 2e-2, ("up projection", it, eh)
        # Partial sums cross NVLink as bf16, so an output can be off by one bf16 step of a partial (which is
        # larger than the output where partials cancel): the bound is relative to the largest output.
        err = ((out.float() - ref).abs().max() / ref.abs().max()).item()
        assert err < 1e-2, ("ffn output", it, err)
    comm.finalize(); comm.destroy()


def symmetry_check():
    """MCCL_CHECK_SYMMETRY=1: calls that keep the contract pass, a send buffer at a rank-dependent offset of a
    symmetric allocation is reported as invalid usage."""
    comm = make_comm()
    k = 4096
    sym = comm.empty(k * WORLD, torch.float32)
    out = comm.empty(k * WORLD, torch.float32)
    sym.copy_(gen(RANK, k * WORLD, torch.float32))
    comm.all_reduce(sym, out, op="sum")
    comm.all_gather(out[RANK * k:(RANK + 1) * k], out)               # in place: the same part by contract
    comm.reduce_scatter(sym, sym[RANK * k:(RANK + 1) * k], op="sum")    # in place
    plain = torch.ones(100, device=DEV)
    comm.all_reduce(plain)
    torch.cuda.synchronize()
    assert comm.async_error() == L.SUCCESS
    comm.all_gather(sym[RANK * k:(RANK + 1) * k], out)               # out of place, offset depends on the rank: refused
    torch.cuda.synchronize()
    assert comm.async_error() == L.INVALID_USAGE, comm.async_error()
    try:
        comm.all_reduce(plain)
        raise AssertionError("the communicator must refuse work after a contract violation")
    except mccl.MCCLError as exc:
        assert exc.code == L.INVALID_USAGE
    comm.host_barrier()
    comm.destroy()


def grouped_allreduce():
    """A group of all-reduce calls goes out as one launch: results against the oracle, the launch count, a group with
    a call that cannot be fused, a group that names two streams, and a timing of 8 x 1 MB grouped against one by one."""
    comm = make_comm()
    cases = [(torch.float32, 4096, "sum"), (torch.bfloat16, 70000, "avg"), (torch.int32, 1 << 16, "max"),
             (torch.float16, 8 * WORLD, "min"), (torch.bfloat16, (1 << 20) + 8, "sum"), (torch.float32, 1 << 18, "avg"),
             (torch.float64, 1024, "sum"), (torch.int64, 2048, "sum")]
    for rep in range(3):                                  # repeated groups reuse flags and counters
        bufs = []
        for dtype, n, op in cases:
            b = comm.empty(n, dtype)
            b.copy_(gen(RANK, n, dtype))
            bufs.append(b)
        torch.cuda.synchronize(); comm.host_barrier()
        before = comm.launch_count
        with mccl.group():
            for b, (dtype, n, op) in zip(bufs, cases):
                comm.all_reduce(b, op=op)
        assert comm.launch_count == before + 1, ("launches for one group", comm.launch_count - before)
        torch.cuda.synchronize()
        assert canary_ok(comm)
        for b, (dtype, n, op) in zip(bufs, cases):
            check(("grouped", rep, dtype, n, op), b, oracle(n, dtype, op), dtype)
            comm.free_raw(b.data_ptr())
    # out of place, plus one call on an ordinary tensor, which takes its own launch after the fused one
    a_in, a_out = comm.empty(5000, torch.float32), comm.empty(5000, torch.float32)
    b_sym = comm.empty(3000, torch.bfloat16)
    plain = torch.empty(777, device=DEV, dtype=torch.float32)
    a_in.copy_(gen(RANK, 5000, torch.float32)); b_sym.copy_(gen(RANK, 3000, torch.bfloat16)); plain.copy_(gen(RANK, 777, torch.float32))
    keep = a_in.clone()
    torch.cuda.synchronize(); comm.host_barrier()
    before = comm.launch_count
    with mccl.group():
        comm.all_reduce(a_in, a_out, op="sum")
        comm.all_reduce(plain, op="sum")
        comm.all_reduce(b_sym, op="avg")
    torch.cuda.synchronize()
    assert comm.launch_count > before + 1
    assert torch.equal(a_in, keep)
    check("grouped out of place", a_out, oracle(5000, torch.float32, "sum"), torch.float32)
    check("grouped, own launch", plain, oracle(777, torch.float32, "sum"), torch.float32)
    check("grouped bf16 avg", b_sym, oracle(3000, torch.bfloat16, "avg"), torch.bfloat16)
    # two streams in one group are refused and leave the communicator usable
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    try:
        with mccl.group():
            comm.all_reduce(a_out, op="sum", stream=s1)
            comm.all_reduce(b_sym, op="sum", stream=s2)
        raise AssertionError("a group with two streams must be refused")
    except mccl.MCCLError as exc:
        assert exc.code == L.INVALID_USAGE, exc.code
    torch.cuda.synchronize(); comm.host_barrier()
    # timing: 8 x 1 MB bf16, grouped against one by one
    k, n = 8, (1 << 20) // 2
    bufs = [comm.empty(n, torch.bfloat16) for _ in range(k)]
    for b in bufs:
        b.normal_()

    def one_by_one():
        for b in bufs:
            comm.all_reduce(b, op="sum")

    def grouped():
        with mccl.group():
            for b in bufs:
                comm.all_reduce(b, op="sum")

    times = {}
    for name, fn in (("one_by_one", one_by_one), ("grouped", grouped)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(); comm.host_barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            fn()
        e1.record(); torch.cuda.synchronize()
        times[name] = e0.elapsed_time(e1) / 20 * 1e3
    if RANK == 0:
        print(f"GROUP_TIMING world={WORLD} 8x1MB bf16 sum: one by one {times['one_by_one']:.1f} us, grouped {times['grouped']:.1f} us", flush=True)
    assert canary_ok(comm)
    comm.finalize(); comm.destroy()


if __name__ == "__main__":
    globals()[sys.argv[1]]()
