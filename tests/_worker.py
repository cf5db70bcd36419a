"""One rank of a multi-process CPU test (tcp transport).  Scenario name in argv[1]; rank/world/port/args in
the environment (see tests/_mp.py).  Exit code 0 = the rank's checks passed."""
from __future__ import annotations

import json
import os
import sys
import threading
import time

import numpy as np

import mccl_b200 as mccl
from mccl_b200 import _lib as L

RANK = int(os.environ["MCCL_TEST_RANK"])
WORLD = int(os.environ["MCCL_TEST_WORLD"])
PORT = int(os.environ["MCCL_TEST_PORT"])
ARGS = json.loads(os.environ.get("MCCL_TEST_ARGS", "{}"))


def make_comm(blocking=True):
    return mccl.Communicator(WORLD, mccl.unique_id_from_env("127.0.0.1", PORT), RANK, blocking=blocking, transport="tcp")


def data(rank, n, dtype=np.float32):
    rng = np.random.default_rng(rank)
    if np.issubdtype(dtype, np.integer):
        lo, hi = (-100, 100) if np.issubdtype(dtype, np.signedinteger) else (0, 100)
        return rng.integers(lo, hi, n).astype(dtype)
    return rng.uniform(-1, 1, n).astype(dtype)


def ref_reduce(arrs, op):
    acc = arrs[0].astype(np.float64) if arrs[0].dtype.kind == "f" else arrs[0].copy()
    for a in arrs[1:]:
        b = a.astype(np.float64) if a.dtype.kind == "f" else a
        if op in ("sum", "avg"):
            acc = acc + b
        elif op == "prod":
            acc = acc * b
        elif op == "max":
            acc = np.maximum(acc, b)
        else:
            acc = np.minimum(acc, b)
    if op == "avg":
        acc = acc / len(arrs) if arrs[0].dtype.kind == "f" else (np.trunc(acc / len(arrs))).astype(arrs[0].dtype)
    return acc


def close(got, ref, dtype):
    if np.dtype(dtype).kind != "f":
        return np.array_equal(got, ref.astype(dtype))
    tol = {2: 2e-2, 4: 1e-5, 8: 1e-12}[np.dtype(dtype).itemsize]
    return np.max(np.abs(got.astype(np.float64) - ref) / (np.abs(ref) + 1.0)) <= tol * WORLD


# ---- scenarios ---------------------------------------------------------------------------------------------
def baseline_config():
    """The CPU plumbing configuration: 1 Mi fp32 per rank ~U[-1,1] seeded by rank; five collectives against numpy; split."""
    comm = make_comm()
    n = 1 << 20
    xs = [data(r, n) for r in range(WORLD)]
    x = xs[RANK]
    ref = ref_reduce(xs, "sum")
    out = np.empty_like(x)
    comm.all_reduce(x, out)
    assert np.max(np.abs(out - ref) / (np.abs(ref) + 1.0)) < 1e-6
    g = np.empty(n * WORLD, np.float32)
    comm.all_gather(x, g)
    assert np.array_equal(g, np.concatenate(xs))
    blk = n // WORLD
    rs = np.empty(blk, np.float32)
    comm.reduce_scatter(x[: blk * WORLD], rs)
    assert np.max(np.abs(rs - ref[RANK * blk:(RANK + 1) * blk]) / (np.abs(ref[RANK * blk:(RANK + 1) * blk]) + 1.0)) < 1e-6
    b = x.copy() if RANK == 0 else np.zeros_like(x)
    comm.broadcast(b if RANK == 0 else None, b, root=0)
    assert np.array_equal(b, xs[0])
    root = 1 % WORLD
    rd = np.empty_like(x) if RANK == root else None
    comm.reduce(x, rd, root=root)
    if RANK == root:
        assert np.max(np.abs(rd - ref) / (np.abs(ref) + 1.0)) < 1e-6
    sub = comm.split(RANK, 0)             # {0}, {1}, ...: every rank alone
    assert sub.size == 1 and sub.rank == 0
    y = np.full(16, RANK + 1.0, np.float32)
    sub.all_reduce(y)
    assert np.all(y == RANK + 1.0)
    sub.finalize(); sub.destroy()
    comm.finalize(); comm.destroy()


def matrix():
    """Every collective x forced algorithm x a few dtypes/ops/counts (odd counts, in place)."""
    comm = make_comm()
    algos = ARGS.get("algos", ["auto", "ring", "tree", "oneshot"])
    dtypes = [np.dtype(d) for d in ARGS.get("dtypes", ["float32", "int32", "float16", "float64", "uint8", "int64"])]
    counts = ARGS.get("counts", [1, 7, 1000, 4099, 300001])
    for algo in algos:
        with mccl.forced_algo(algo):
            for dt in dtypes:
                for n in counts:
                    xs = [data(r, n, dt) for r in range(WORLD)]
                    for op in ("sum", "max", "avg") if dt.kind == "f" else ("sum", "min", "prod"):
                        if dt.kind != "f" and op == "prod":
                            xs2 = [np.sign(a).astype(dt) if dt.kind == "i" else (a % 2).astype(dt) for a in xs]
                        else:
                            xs2 = xs
                        buf = xs2[RANK].copy()
                        comm.all_reduce(buf, op=op)       # in place
                        assert close(buf, ref_reduce(xs2, op), dt), ("allreduce", algo, dt, n, op)
                    g = np.empty(n * WORLD, dt)
                    g[RANK * n:(RANK + 1) * n] = xs[RANK]
                    comm.all_gather(g[RANK * n:(RANK + 1) * n], g)     # in place slot
                    assert np.array_equal(g, np.concatenate(xs)), ("allgather", algo, dt, n)
                    full = [data(r + 100, n * WORLD, dt) for r in range(WORLD)]
                    o = np.empty(n, dt)
                    comm.reduce_scatter(full[RANK], o, op="sum")
                    assert close(o, ref_reduce(full, "sum")[RANK * n:(RANK + 1) * n], dt), ("reducescatter", algo, dt, n)
                    for root in {0, WORLD - 1}:
                        b = xs[root].copy() if RANK == root else np.zeros(n, dt)
                        comm.broadcast(b if RANK == root else None, b, root=root)
                        assert np.array_equal(b, xs[root]), ("broadcast", algo, dt, n, root)
                        rd = np.empty(n, dt) if RANK == root else None
                        comm.reduce(xs[RANK], rd, op="sum", root=root)
                        if RANK == root:
                            assert close(rd, ref_reduce(xs, "sum"), dt), ("reduce", algo, dt, n, root)
    comm.finalize(); comm.destroy()


def bf16():
    import torch
    comm = make_comm()
    n = 5003
    xs = [torch.from_numpy(data(r, n)).to(torch.bfloat16) for r in range(WORLD)]
    for algo in ("ring", "tree", "oneshot"):
        with mccl.forced_algo(algo):
            buf = xs[RANK].clone()
            comm.all_reduce(buf, op="avg")
            ref = torch.stack([x.double() for x in xs]).sum(0) / WORLD
            assert ((buf.double() - ref).abs() / (ref.abs() + 1)).max() < 3e-2 * WORLD, algo
    comm.finalize(); comm.destroy()


def p2p_group():
    comm = make_comm()
    n = 100003
    x = data(RANK, n)
    y = np.empty_like(x)
    nxt, prv = (RANK + 1) % WORLD, (RANK - 1) % WORLD
    with mccl.group():
        comm.send(x, nxt)
        comm.recv(y, prv)
    assert np.array_equal(y, data(prv, n))
    # all-to-all with provenance tags: value = src * WORLD + dst
    blk = 513
    s = np.repeat(np.arange(WORLD, dtype=np.float32) + RANK * WORLD, blk)
    r = np.empty_like(s)
    comm.all_to_all(s, r)
    exp = np.repeat(np.arange(WORLD, dtype=np.float32) * WORLD + RANK, blk)
    assert np.array_equal(r, exp)
    # RecvAny: every rank but 0 sends one message to rank 0, which collects them in arrival order
    if RANK == 0:
        seen = set()
        for _ in range(WORLD - 1):
            buf = np.empty(64, np.float32)
            src = comm.recv_any(buf)
            assert np.all(buf == float(src)), (src, buf[:4])
            seen.add(src)
        assert seen == set(range(1, WORLD))
    else:
        comm.send(np.full(64, float(RANK), np.float32), 0)
    # a collective recorded inside a group runs at GroupEnd
    z = np.full(8, 1.0, np.float32)
    with mccl.group():
        comm.all_reduce(z)
    assert np.all(z == WORLD)
    comm.finalize(); comm.destroy()


def stripe_integrity():
    """Byte-pattern transfers around the striping threshold with several sockets per connection (the reference's
    MCCL_M2M_MAIN check: data[i] == i & 0xff on arrival)."""
    comm = make_comm()
    peer = 1 - RANK
    for nbytes in (1, 4095, 256 * 1024 - 1, 256 * 1024, 256 * 1024 + 1, 3 * 1024 * 1024 + 7):
        pattern = (np.arange(nbytes, dtype=np.uint32) & 0xFF).astype(np.uint8)
        got = np.zeros(nbytes, np.uint8)
        with mccl.group():
            comm.send(pattern, peer)
            comm.recv(got, peer)
        assert np.array_equal(got, pattern), nbytes
    comm.finalize(); comm.destroy()


def nonblocking():
    comm = make_comm(blocking=False)
    n = 1 << 18
    bufs = [data(RANK + 10 * i, n) for i in range(4)]
    outs = [np.empty(n, np.float32) for _ in range(4)]
    for b, o in zip(bufs, outs):
        comm.all_reduce(b, o)                 # returns at once, work runs on the communicator's thread
    saw_progress = comm.async_error() in (L.SUCCESS, L.IN_PROGRESS)
    comm.synchronize()
    assert saw_progress and comm.async_error() == L.SUCCESS
    for i, o in enumerate(outs):
        ref = ref_reduce([data(r + 10 * i, n) for r in range(WORLD)], "sum")
        assert close(o, ref, np.float32)
    comm.finalize(); comm.destroy()


def split_groups():
    comm = make_comm()
    color = RANK % 2
    sub = comm.split(color, key=-RANK)        # reversed order inside each group
    members = [r for r in range(WORLD) if r % 2 == color]
    assert sub.size == len(members)
    assert sub.rank == sorted(members, key=lambda r: -r).index(RANK)
    y = np.full(32, RANK + 1.0, np.float32)
    sub.all_reduce(y)
    assert np.all(y == sum(r + 1.0 for r in members))
    none = comm.split(mccl.SPLIT_NOCOLOR if RANK == 0 else 5, 0)
    assert (none is None) == (RANK == 0)
    if none is not None:
        assert none.size == WORLD - 1
        none.finalize(); none.destroy()
    sub.finalize(); sub.destroy()
    comm.finalize(); comm.destroy()


def usage_errors():
    comm = make_comm()
    lib = L.load()
    x = np.zeros(8, np.float32)
    import ctypes as C
    h = C.c_void_p(comm.handle)
    assert lib.mcclAllReduce(h, None, x.ctypes.data, 8, L.FLOAT32, L.SUM, None) == L.INVALID_ARGUMENT
    assert lib.mcclAllReduce(h, x.ctypes.data, x.ctypes.data, 8, 99, L.SUM, None) == L.INVALID_ARGUMENT
    assert lib.mcclAllReduce(h, x.ctypes.data, x.ctypes.data, 8, L.FLOAT32, 17, None) == L.INVALID_ARGUMENT
    assert lib.mcclAllReduce(h, None, None, 0, L.FLOAT32, L.SUM, None) == L.SUCCESS        # count 0: no-op
    assert lib.mcclBroadcast(h, x.ctypes.data, x.ctypes.data, 8, L.FLOAT32, WORLD, None) == L.INVALID_ARGUMENT
    assert lib.mcclSend(h, x.ctypes.data, 8, L.FLOAT32, WORLD + 3, None) == L.INVALID_ARGUMENT
    assert lib.mcclGroupEnd() == L.INVALID_USAGE
    # usage errors do not poison the communicator
    comm.all_reduce(x)
    assert comm.async_error() == L.SUCCESS
    comm.finalize(); comm.destroy()


def abort_unblocks():
    """Rank 0 parks in a receive nobody will satisfy; a second thread aborts; the call returns an error."""
    comm = make_comm()
    comm.host_barrier()
    if RANK == 0:
        err = {}

        def park():
            try:
                comm.recv(np.empty(1 << 16, np.float32), 1 % WORLD)
                err["rc"] = "returned"
            except mccl.MCCLError as e:
                err["rc"] = e.code
        t = threading.Thread(target=park)
        t.start()
        time.sleep(0.5)
        comm.abort()
        t.join(timeout=20)
        assert not t.is_alive(), "abort did not unblock the receive"
        assert err.get("rc") not in (None, "returned"), err
        assert comm.async_error() == L.INVALID_USAGE
    else:
        time.sleep(1.5)
        comm.abort()
    # aborted communicators are destroyed without a finalize barrier
    comm.destroy()


def peer_dies():
    """Rank 1 exits before the collective; the others get an error (not a hang) and the error is sticky."""
    comm = make_comm()
    comm.host_barrier()
    if RANK == 1:
        os._exit(0)
    time.sleep(0.3)
    x = np.ones(1 << 20, np.float32)
    try:
        comm.all_reduce(x)
        raise SystemExit("all_reduce with a dead peer returned success")
    except mccl.MCCLError as e:
        assert e.code in (L.SYSTEM_ERROR, L.REMOTE_ERROR), e.code
    assert comm.async_error() in (L.SYSTEM_ERROR, L.REMOTE_ERROR)
    try:
        comm.all_reduce(x)
        raise SystemExit("second call on a failed communicator returned success")
    except mccl.MCCLError as e:
        assert e.code in (L.SYSTEM_ERROR, L.REMOTE_ERROR)
    comm.abort(); comm.destroy()


def recover_smaller():
    """Recovery as the library defines it (abort, destroy, initialise again): the last rank leaves between two steps,
    the survivors' next collective fails instead of hanging, they drop the communicator, meet again as a smaller world
    on a second rendezvous port, restore the optimizer state saved before the failure and keep training in step."""
    import io
    import torch
    from mccl_b200.models.gpt2 import GPT2, GPT2Config
    from mccl_b200.parallel.ddp import DistributedDataParallel
    comm = make_comm()
    cfg = GPT2Config.tiny()
    torch.manual_seed(0)
    ddp = DistributedDataParallel(GPT2(cfg), comm, bucket_mb=0.25)
    g = torch.Generator().manual_seed(31 + RANK)
    t = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len + 1), generator=g)
    ddp(t[:, :-1], t[:, 1:]).backward(); ddp.step(lr=1e-3)
    blob = io.BytesIO()
    torch.save(ddp.optimizer_state_dict(), blob)                   # the checkpoint every rank keeps
    comm.host_barrier()
    if RANK == WORLD - 1:
        os._exit(0)                                                # leaves between steps, nothing in flight
    time.sleep(0.3)
    try:
        ddp(t[:, :-1], t[:, 1:]).backward(); ddp.step(lr=1e-3)
        raise SystemExit("a step with a dead peer returned success")
    except mccl.MCCLError as e:
        assert e.code in (L.SYSTEM_ERROR, L.REMOTE_ERROR), e.code
    comm.abort(); comm.destroy()
    small = mccl.Communicator(WORLD - 1, mccl.unique_id_from_env("127.0.0.1", ARGS["port2"]), RANK, transport="tcp")
    torch.manual_seed(99)
    again = DistributedDataParallel(GPT2(cfg), small, bucket_mb=0.25)
    blob.seek(0)
    again.load_optimizer_state_dict(torch.load(blob))
    for _ in range(2):
        again(t[:, :-1], t[:, 1:]).backward(); again.step(lr=1e-3)
    import hashlib
    h = hashlib.sha256()
    for b in again.buckets:
        h.update(b.param.numpy().tobytes())
    digests = small.host_all_gather(h.digest())
    assert all(d == digests[0] for d in digests), "survivors diverged after the restart"
    small.finalize(); small.destroy()


def never_joins():
    """Rank WORLD-1 never calls init: everyone else fails the rendezvous within the deadline."""
    if RANK == WORLD - 1:
        return
    t0 = time.time()
    try:
        make_comm()
        raise SystemExit("init succeeded without the last rank")
    except mccl.MCCLError as e:
        assert e.code in (L.SYSTEM_ERROR, L.REMOTE_ERROR), e.code
    assert time.time() - t0 < 30


def inject_socket_fault():
    """MCCL_FAULT_INJECT=send:N on rank 0 makes its Nth socket send fail: the collective reports a fatal error."""
    comm = make_comm()
    x = np.ones(1 << 16, np.float32)
    failed = False
    for _ in range(6):
        try:
            comm.all_reduce(x.copy())
        except mccl.MCCLError as e:
            assert e.code in (L.SYSTEM_ERROR, L.REMOTE_ERROR)
            failed = True
            break
    assert failed, "the injected fault never surfaced"
    comm.abort(); comm.destroy()


def ddp_cpu():
    """Two-process DDP on the tcp transport equals single-process training on the concatenated batch."""
    import torch
    from mccl_b200.models.gpt2 import GPT2, GPT2Config
    from mccl_b200.parallel.ddp import DistributedDataParallel
    comm = make_comm()
    torch.manual_seed(17 * RANK)               # replicas seeded apart: the wrapper must start them from rank 0's weights
    cfg = GPT2Config.tiny()
    model = GPT2(cfg)
    ddp = DistributedDataParallel(model, comm, bucket_mb=0.25)
    assert len(ddp.buckets) > 2
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, cfg.vocab_size, (2 * WORLD, cfg.seq_len + 1), generator=g)
    mine = tokens[2 * RANK: 2 * RANK + 2]
    torch.manual_seed(0)
    single = GPT2(cfg)
    ref = DistributedDataParallel(single, None, bucket_mb=0.25)
    for (n1, p1), (n2, p2) in zip(model.named_parameters(), single.named_parameters()):
        assert torch.equal(p1, p2), ("initial parameters differ from rank 0's", n1)
    # gradients of the first step: the bucket all-reduce (avg) must reproduce the global-batch gradient
    loss = ddp(mine[:, :-1], mine[:, 1:]); loss.backward(); ddp.finish_backward()
    l2 = ref(tokens[:, :-1], tokens[:, 1:]); l2.backward()
    for (n1, p1), (n2, p2) in zip(model.named_parameters(), single.named_parameters()):
        assert torch.allclose(p1.grad, p2.grad, atol=1e-6, rtol=1e-4), (n1, (p1.grad - p2.grad).abs().max().item())
    ddp.step(lr=1e-3); ref.step(lr=1e-3)
    for _ in range(2):
        loss = ddp(mine[:, :-1], mine[:, 1:]); loss.backward(); ddp.step(lr=1e-3)
        l2 = ref(tokens[:, :-1], tokens[:, 1:]); l2.backward(); ref.step(lr=1e-3)
    # Adam divides by sqrt(v): elements with near-zero gradients amplify rounding, so the bound is a
    # fraction of the total possible movement (3 steps x lr).
    for (n1, p1), (n2, p2) in zip(model.named_parameters(), single.named_parameters()):
        assert (p1 - p2).abs().max().item() < 1.5e-3, (n1, (p1 - p2).abs().max().item())
        assert (p1 - p2).abs().mean().item() < 5e-5, (n1, (p1 - p2).abs().mean().item())
    comm.finalize(); comm.destroy()


def ddp_zero():
    """Sharded optimizer (reduce-scatter, update of the own slice, all-gather): the parameters follow
    single-process training on the concatenated batch, on every rank alike, and the optimizer state is 1/world."""
    import torch
    from mccl_b200.models.gpt2 import GPT2, GPT2Config
    from mccl_b200.parallel.ddp import DistributedDataParallel
    comm = make_comm()
    torch.manual_seed(0)
    cfg = GPT2Config.tiny()
    model = GPT2(cfg)
    ddp = DistributedDataParallel(model, comm, bucket_mb=0.25, shard_optimizer=True)
    assert len(ddp.buckets) > 2
    for b in ddp.buckets:
        assert b.numel % (8 * WORLD) == 0 and b.master.numel() == b.numel // WORLD == b.exp_avg.numel()
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, cfg.vocab_size, (2 * WORLD, cfg.seq_len + 1), generator=g)
    mine = tokens[2 * RANK: 2 * RANK + 2]
    torch.manual_seed(0)
    single = GPT2(cfg)
    ref = DistributedDataParallel(single, None, bucket_mb=0.25)
    for _ in range(3):
        loss = ddp(mine[:, :-1], mine[:, 1:]); loss.backward(); ddp.step(lr=1e-3)
        l2 = ref(tokens[:, :-1], tokens[:, 1:]); l2.backward(); ref.step(lr=1e-3)
    for (n1, p1), (n2, p2) in zip(model.named_parameters(), single.named_parameters()):
        assert (p1 - p2).abs().max().item() < 1.5e-3, (n1, (p1 - p2).abs().max().item())
        assert (p1 - p2).abs().mean().item() < 5e-5, (n1, (p1 - p2).abs().mean().item())
        assert p1.grad.abs().max().item() == 0.0, n1                 # cleared for the next accumulation
    # every rank holds the same parameters, bit for bit
    import hashlib
    h = hashlib.sha256()
    for b in ddp.buckets:
        h.update(b.param.numpy().tobytes())
    digests = comm.host_all_gather(h.digest())
    assert all(d == digests[0] for d in digests)
    comm.finalize(); comm.destroy()


def c10d_backend():
    """The "mccl" torch.distributed backend on cpu tensors (tcp transport): the c10d calls torch code makes, then
    torch's own DistributedDataParallel on top of it against single-process training."""
    import torch
    import torch.distributed as dist
    import mccl_b200.c10d  # noqa: F401  (registers the backend)
    dist.init_process_group("mccl", rank=RANK, world_size=WORLD, init_method="file://" + ARGS["rendezvous"])
    assert dist.get_backend() == "mccl"
    n = WORLD
    t = torch.full((1000,), RANK + 1.0)
    dist.all_reduce(t)
    assert torch.all(t == n * (n + 1) / 2)
    t = torch.full((7,), RANK + 1.0, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert torch.all(t == n)
    w = dist.all_reduce(torch.ones(5), async_op=True)
    w.wait()
    assert w.is_completed()
    b = torch.arange(10, dtype=torch.int64) * (1 if RANK == 1 else 0)
    dist.broadcast(b, src=1)
    assert torch.equal(b, torch.arange(10, dtype=torch.int64))
    out = torch.empty(4 * n)
    dist.all_gather_into_tensor(out, torch.full((4,), float(RANK)))
    assert torch.equal(out, torch.arange(n, dtype=torch.float32).repeat_interleave(4))
    outs = [torch.empty(3, 2) for _ in range(n)]
    dist.all_gather(outs, torch.full((3, 2), float(RANK)))
    assert all(torch.all(o == r) for r, o in enumerate(outs))
    rs = torch.empty(5)
    dist.reduce_scatter_tensor(rs, torch.arange(5 * n, dtype=torch.float32), op=dist.ReduceOp.SUM)
    assert torch.equal(rs, n * torch.arange(5 * RANK, 5 * RANK + 5, dtype=torch.float32))
    r = torch.full((6,), RANK + 1.0)
    dist.reduce(r, dst=0, op=dist.ReduceOp.SUM)
    assert RANK != 0 or torch.all(r == n * (n + 1) / 2)
    a2a = torch.empty(2 * n)
    dist.all_to_all_single(a2a, torch.arange(2 * n, dtype=torch.float32) + 100 * RANK)
    assert torch.equal(a2a, torch.cat([torch.arange(2 * RANK, 2 * RANK + 2, dtype=torch.float32) + 100 * s for s in range(n)]))
    got = [torch.empty(5) for _ in range(n)] if RANK == n - 1 else None
    dist.gather(torch.full((5,), float(RANK)), got, dst=n - 1)
    assert RANK != n - 1 or all(torch.all(t == float(p)) for p, t in enumerate(got))
    piece = torch.empty(4)
    dist.scatter(piece, [torch.full((4,), 10.0 + p) for p in range(n)] if RANK == 0 else None, src=0)
    assert torch.all(piece == 10.0 + RANK)
    # unequal splits: rank r sends (j + 1) rows to rank j and receives (r + 1) rows from everyone
    rows_in = torch.cat([torch.full((j + 1, 3), float(100 * RANK + j)) for j in range(n)])
    rows_out = torch.empty(n * (RANK + 1), 3)
    dist.all_to_all_single(rows_out, rows_in, output_split_sizes=[RANK + 1] * n, input_split_sizes=[j + 1 for j in range(n)])
    assert torch.equal(rows_out, torch.cat([torch.full((RANK + 1, 3), float(100 * s + RANK)) for s in range(n)]))
    if RANK == 0:
        dist.send(torch.full((9,), 3.5), dst=1)
    elif RANK == 1:
        got = torch.zeros(9)
        dist.recv(got, src=0)
        assert torch.all(got == 3.5)
    dist.barrier()
    sub = dist.new_group([0, n - 1])                       # a subgroup gets its own communicator
    if RANK in (0, n - 1):
        t = torch.full((11,), RANK + 1.0)
        dist.all_reduce(t, group=sub)
        assert torch.all(t == (1.0 + n if n > 1 else 1.0)), t
    comm = dist.group.WORLD.communicator("cpu")
    assert comm.size == n and comm.rank == RANK and comm.transport == "tcp"
    with pytest_raises(ValueError):
        dist.all_reduce(torch.ones(3, dtype=torch.int32), op=dist.ReduceOp.BXOR)

    # DTensor on a device mesh over the backend: redistribution (all-gather) and a sharded matmul (partial sums reduced)
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Replicate, Shard, distribute_tensor
    mesh = init_device_mesh("cpu", (n,))
    torch.manual_seed(0)
    full, w = torch.randn(4 * n, 2 * n), torch.randn(2 * n, 5)
    assert torch.equal(distribute_tensor(full, mesh, [Shard(0)]).redistribute(mesh, [Replicate()]).to_local(), full)
    y = torch.matmul(distribute_tensor(full, mesh, [Shard(1)]), distribute_tensor(w, mesh, [Shard(0)]))
    assert torch.allclose(y.redistribute(mesh, [Replicate()]).to_local(), full @ w, atol=1e-5)

    # torch DDP on top of the backend
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))
    ref = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))
    ref.load_state_dict(net.state_dict())
    ddp = torch.nn.parallel.DistributedDataParallel(net, bucket_cap_mb=0.001)
    g = torch.Generator().manual_seed(3)
    x, y = torch.randn(4 * n, 16, generator=g), torch.randn(4 * n, 4, generator=g)
    o1, o2 = torch.optim.SGD(ddp.parameters(), lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    for _ in range(3):
        o1.zero_grad(); torch.nn.functional.mse_loss(ddp(x[4 * RANK:4 * RANK + 4]), y[4 * RANK:4 * RANK + 4]).backward(); o1.step()
        o2.zero_grad(); torch.nn.functional.mse_loss(ref(x), y).backward(); o2.step()
    for p1, p2 in zip(net.parameters(), ref.parameters()):
        assert torch.allclose(p1, p2, atol=1e-6, rtol=1e-5), (p1 - p2).abs().max().item()

    # torch FSDP2 (fully_shard: parameters as DTensors, all-gather / reduce-scatter per layer) on top of the backend
    from torch.distributed.fsdp import fully_shard
    torch.manual_seed(1)
    fs = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))
    ref = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))
    ref.load_state_dict(fs.state_dict())
    for layer in (fs[0], fs[2]):
        fully_shard(layer, mesh=mesh)
    fully_shard(fs, mesh=mesh)
    o1, o2 = torch.optim.SGD(fs.parameters(), lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    for _ in range(3):
        o1.zero_grad(); torch.nn.functional.mse_loss(fs(x[4 * RANK:4 * RANK + 4]), y[4 * RANK:4 * RANK + 4]).backward(); o1.step()
        o2.zero_grad(); torch.nn.functional.mse_loss(ref(x), y).backward(); o2.step()
    for p1, p2 in zip(fs.parameters(), ref.parameters()):
        assert torch.allclose(p1.full_tensor(), p2, atol=1e-5, rtol=1e-4), (p1.full_tensor() - p2).abs().max().item()
    dist.destroy_process_group()


class pytest_raises:
    def __init__(self, exc):
        self.exc = exc

    def __enter__(self):
        return self

    def __exit__(self, et, ev, tb):
        assert et is not None and issubclass(et, self.exc), f"expected {self.exc}, got {et}"
        return True


def parallel_layers():
    import torch
    from _parallel_cases import layers_case
    comm = make_comm()
    layers_case(comm, RANK, WORLD, torch.device("cpu"))
    comm.finalize(); comm.destroy()


def llama_tp():
    import torch
    from _parallel_cases import llama_case
    comm = make_comm()
    llama_case(comm, RANK, WORLD, torch.device("cpu"))
    comm.finalize(); comm.destroy()


def tp_dp_2d():
    """Four ranks as tensor parallel 2 x data parallel 2 (two splits of the world communicator): the Llama-style model
    on the tensor-parallel group inside the bucketed DDP wrapper on the data-parallel group reproduces the
    single-process gradient of the whole batch."""
    import torch
    import mccl_b200 as mccl
    from mccl_b200.models.llama import Llama, LlamaConfig
    from mccl_b200.parallel.ddp import DistributedDataParallel
    world = make_comm()
    assert WORLD == 4
    tp = world.split(RANK // 2, RANK)            # ranks {0,1} and {2,3}
    dp = world.split(RANK % 2, RANK)             # ranks {0,2} and {1,3}
    assert tp.size == 2 and dp.size == 2 and tp.rank == RANK % 2 and dp.rank == RANK // 2
    cfg = LlamaConfig.tiny()
    one = mccl.Communicator(1, mccl.get_unique_id(), 0, transport="tcp")
    torch.manual_seed(0)
    ref = Llama(cfg, one)
    state = {k: v.detach().clone() for k, v in ref.named_parameters()}
    g = torch.Generator().manual_seed(4)
    tokens = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len + 1), generator=g)
    ref(tokens[:, :-1], tokens[:, 1:]).backward()
    model = Llama(cfg, tp)
    model.load_full(state)
    ddp = DistributedDataParallel(model, dp, bucket_mb=0.05)
    mine = tokens[2 * dp.rank: 2 * dp.rank + 2]  # each data-parallel replica takes half of the batch
    ddp(mine[:, :-1], mine[:, 1:]).backward()
    ddp.finish_backward()
    full = dict(ref.named_parameters())
    for name, p in model.named_parameters():
        want = full[name].grad
        leaf = name.split(".")[-2]
        if leaf in ("q", "k", "v", "gate", "up"):
            m = want.shape[0] // 2
            want = want[tp.rank * m:(tp.rank + 1) * m]
        elif leaf in ("o", "down"):
            m = want.shape[1] // 2
            want = want[:, tp.rank * m:(tp.rank + 1) * m]
        assert torch.allclose(p.grad, want, atol=2e-5, rtol=1e-3), (name, (p.grad - want).abs().max().item())
    for c in (tp, dp):
        c.finalize(); c.destroy()
    one.destroy()
    world.finalize(); world.destroy()


def pipeline_1f1b():
    import torch
    from _parallel_cases import pipeline_case
    comm = make_comm()
    pipeline_case(comm, RANK, WORLD, torch.device("cpu"), atol=1e-6)
    comm.finalize(); comm.destroy()


def ddp_checkpoint():
    """Save after two steps, continue for two more; a fresh wrapper that loads the checkpoint and runs the same two
    steps ends with bit-identical parameters (replicated and sharded optimizer)."""
    import io
    import torch
    from mccl_b200.models.gpt2 import GPT2, GPT2Config
    from mccl_b200.parallel.ddp import DistributedDataParallel
    comm = make_comm()
    cfg = GPT2Config.tiny()
    g = torch.Generator().manual_seed(21 + RANK)
    batches = [torch.randint(0, cfg.vocab_size, (2, cfg.seq_len + 1), generator=g) for _ in range(4)]
    for shard in (False, True):
        torch.manual_seed(0)
        ddp = DistributedDataParallel(GPT2(cfg), comm, bucket_mb=0.25, shard_optimizer=shard)
        def run(d, bs):
            for t in bs:
                d(t[:, :-1], t[:, 1:]).backward(); d.step(lr=1e-3)
        run(ddp, batches[:2])
        blob = io.BytesIO()
        torch.save(ddp.optimizer_state_dict(), blob)
        run(ddp, batches[2:])
        torch.manual_seed(123)                                    # different initial weights: everything comes from the file
        again = DistributedDataParallel(GPT2(cfg), comm, bucket_mb=0.25, shard_optimizer=shard)
        blob.seek(0)
        again.load_optimizer_state_dict(torch.load(blob))
        assert again.step_count == 2
        run(again, batches[2:])
        for b1, b2 in zip(ddp.buckets, again.buckets):
            assert torch.equal(b1.param, b2.param) and torch.equal(b1.master, b2.master), (shard, "diverged after resume")
    comm.finalize(); comm.destroy()


def fsdp_stack():
    import torch
    from _parallel_cases import fsdp_case
    comm = make_comm()
    fsdp_case(comm, RANK, WORLD, torch.device("cpu"))
    comm.finalize(); comm.destroy()


def rooted_and_ragged():
    """mcclGather, mcclScatter and mcclAllToAllv (compositions of grouped Send / Recv) on the tcp transport."""
    comm = make_comm()
    n, r = WORLD, RANK
    for root in (0, n - 1):
        out = np.zeros(5 * n, np.float32) if r == root else None
        comm.gather(np.full(5, float(r), np.float32), out, root=root)
        if r == root:
            assert np.array_equal(out, np.repeat(np.arange(n, dtype=np.float32), 5))
        piece = np.zeros(3, np.int64)
        comm.scatter(np.arange(3 * n, dtype=np.int64) if r == root else None, piece, root=root)
        assert np.array_equal(piece, np.arange(3 * r, 3 * r + 3))
    # rank r sends j + 1 elements to rank j (value 100 r + j) and receives r + 1 from everyone
    send = np.concatenate([np.full(j + 1, 100.0 * r + j) for j in range(n)]).astype(np.float64)
    recv = np.zeros(n * (r + 1), np.float64)
    comm.all_to_all_v(send, [j + 1 for j in range(n)], recv, [r + 1] * n)
    assert np.array_equal(recv, np.concatenate([np.full(r + 1, 100.0 * s + r) for s in range(n)]))
    # zero-length segments
    send = np.full(4, float(r), np.float32)
    recv = np.zeros(4 if r == 0 else 0, np.float32) if n == 1 else np.zeros(4 * n if r == 0 else 0, np.float32)
    comm.all_to_all_v(send, [4] + [0] * (n - 1), recv, [4] * n if r == 0 else [0] * n)
    if r == 0:
        assert np.array_equal(recv, np.repeat(np.arange(n, dtype=np.float32), 4))
    comm.finalize(); comm.destroy()


def ddp_accumulate():
    """Two micro-batches (the first under no_sync) give the gradient of the concatenated batch."""
    import torch
    from mccl_b200.models.gpt2 import GPT2, GPT2Config
    from mccl_b200.parallel.ddp import DistributedDataParallel
    comm = make_comm()
    torch.manual_seed(0)
    cfg = GPT2Config.tiny()
    model = GPT2(cfg)
    ddp = DistributedDataParallel(model, comm, bucket_mb=0.25)
    g = torch.Generator().manual_seed(11)
    tokens = torch.randint(0, cfg.vocab_size, (4 * WORLD, cfg.seq_len + 1), generator=g)
    mine = tokens[4 * RANK: 4 * RANK + 4]
    before = comm.launch_count
    with ddp.no_sync():
        (ddp(mine[:2, :-1], mine[:2, 1:]) / 2).backward()
    (ddp(mine[2:, :-1], mine[2:, 1:]) / 2).backward()
    ddp.finish_backward()
    torch.manual_seed(0)
    single = GPT2(cfg)
    single(tokens[:, :-1], tokens[:, 1:]).backward()
    for (n1, p1), (n2, p2) in zip(model.named_parameters(), single.named_parameters()):
        assert torch.allclose(p1.grad, p2.grad, atol=2e-6, rtol=1e-4), (n1, (p1.grad - p2.grad).abs().max().item())
    comm.finalize(); comm.destroy()


if __name__ == "__main__":
    globals()[sys.argv[1]]()
