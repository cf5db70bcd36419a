"""Command-line probes, one per subsystem (the role of the reference's `#ifdef MCCL_*_MAIN` programs:
allocator, trees, connect, xml, utils, metal, init, m2m, bootstrap, discover, comm, coll).

    python -m mccl_b200.probe alloc [--size 65536 --count 4]
    python -m mccl_b200.probe trees [--max 256]
    python -m mccl_b200.probe connect [--nodes 16] [--cuda]
    python -m mccl_b200.probe xml [--nodes 8] [--cuda] [--out topo.xml]
    python -m mccl_b200.probe gpu                      # device facts, exit 1 if the GPU is not sm_100
    python -m mccl_b200.probe kernels                  # single-GPU checks of the reduction kernels
    python -m mccl_b200.probe comm                     # rank/world from MCCL_RANK / MCCL_WORLD_SIZE (or RANK / WORLD_SIZE)
    python -m mccl_b200.probe coll --op allreduce|allgather|reducescatter|broadcast|reduce|alltoall [--count N --root R]
    python -m mccl_b200.probe bw [--mbytes 256]        # measured pair bandwidth / empty-collective latency (cuda transport)
    python -m mccl_b200.probe bootstrap                # control-plane all-gather of 1000 + rank
    python -m mccl_b200.probe m2m [--bytes 8388608]    # striped TCP transfer rank 0 -> 1 with a byte-pattern check
    python -m mccl_b200.probe discover                 # what discovery found: ranks, links, NVLS, per-algorithm plans

Distributed probes read MCCL_RANK, MCCL_WORLD_SIZE, MCCL_BOOTSTRAP_IP and MCCL_BOOTSTRAP_PORT (defaults
0, 1, 127.0.0.1, 53700), like the reference's launch convention (README.md:29-31).  Exit code 0 = pass.
"""
from __future__ import annotations

import argparse
import ctypes as C
import os
import sys

import numpy as np

from . import _lib as L
from .comm import Communicator, get_unique_id, unique_id_from_env


def _env_world():
    rank = int(os.environ.get("MCCL_RANK", os.environ.get("RANK", "0")))
    world = int(os.environ.get("MCCL_WORLD_SIZE", os.environ.get("WORLD_SIZE", "1")))
    ip = os.environ.get("MCCL_BOOTSTRAP_IP", "127.0.0.1")
    port = int(os.environ.get("MCCL_BOOTSTRAP_PORT", "53700"))
    return rank, world, ip, port


def _comm(transport=None):
    rank, world, ip, port = _env_world()
    if transport == "cuda" or (transport is None and os.environ.get("MCCL_TRANSPORT", "") == "cuda"):
        # one GPU per rank: the local rank of the launcher, else the rank itself
        import torch
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)) % max(torch.cuda.device_count(), 1))
    return Communicator(world, unique_id_from_env(ip, port), rank, transport=transport)


def probe_alloc(a) -> int:
    lib = L.load()
    pool = C.c_void_p()
    L.check(lib.mcclMemPoolCreate(a.size, a.count, C.byref(pool)))
    bufs = []
    for _ in range(a.count + 1):                      # one more than the pool holds: it must grow
        b = L.Buf()
        L.check(lib.mcclMemPoolAlloc(pool, C.byref(b)))
        bufs.append(b)
    page = os.sysconf("SC_PAGESIZE")
    ok = all(b.host % page == 0 for b in bufs) and len({b.host for b in bufs}) == len(bufs)
    L.check(lib.mcclMemPoolFree(pool, C.byref(bufs[0])))
    again = L.Buf()
    L.check(lib.mcclMemPoolAlloc(pool, C.byref(again)))
    ok = ok and again.host == bufs[0].host
    lib.mcclMemPoolDestroy(pool)
    print(f"alloc: {len(bufs)} page-aligned buffers of {a.size} bytes, pool grew and reused: {'ok' if ok else 'FAIL'}")
    return 0 if ok else 1


def probe_trees(a) -> int:
    lib = L.load()
    bad = 0
    for n in range(1, a.max + 1):
        t = []
        for r in range(n):
            out = (C.c_int * 6)()
            lib.mcclDbgDtree(n, r, out)
            t.append(list(out))
        if n > 2:
            leaf_both = [r for r in range(n) if t[r][1] < 0 and t[r][2] < 0 and t[r][4] < 0 and t[r][5] < 0]
            roots = ([r for r in range(n) if t[r][0] < 0], [r for r in range(n) if t[r][3] < 0])
            if leaf_both or roots[0] == roots[1]:
                bad += 1
                print(f"n={n}: leaf in both trees {leaf_both}, roots {roots}")
    print(f"trees: n = 1..{a.max}: {'ok' if not bad else f'{bad} violations'}")
    return 1 if bad else 0


def probe_connect(a) -> int:
    lib = L.load()
    n, cap = a.nodes, 16
    roots, ok = 0, True
    for r in range(n):
        out = (C.c_int * (4 + 2 * (2 + cap)))()
        L.check(lib.mcclDbgSyntheticChannel(n, r, 1 if a.cuda else 0, 0, out, cap))
        v = list(out)
        up, nd = v[4], v[5]
        roots += up < 0
        print(f"rank {r}: ring {v[0]} -> {r} -> {v[1]}  tree up {up} down {v[6:6 + nd]}  flat {v[2]} dtree {v[3]}")
    ok = roots == 1
    print(f"connect: exactly one root: {'ok' if ok else 'FAIL'}")
    return 0 if ok else 1


def probe_xml(a) -> int:
    lib = L.load()
    p = C.c_void_p()
    L.check(lib.mcclDbgSyntheticTopoXml(a.nodes, 1 if a.cuda else 0, C.c_float(0.0), 1 if a.cuda else 0, C.byref(p)))
    s = C.string_at(p).decode()
    lib.mcclFreeString(p)
    if a.out:
        open(a.out, "w").write(s)
    print(s)
    return 0


def probe_gpu(a) -> int:
    import torch
    if not torch.cuda.is_available():
        print("gpu: no CUDA device")
        return 1
    p = torch.cuda.get_device_properties(0)
    print(f"gpu: {p.name} sm_{p.major}{p.minor} {p.multi_processor_count} SMs {p.total_memory / 2**30:.0f} GiB, "
          f"{torch.cuda.device_count()} visible")
    return 0 if p.major == 10 else 1


def probe_kernels(a) -> int:
    """Single-GPU numeric checks of the library's reduction-side kernels (sum of squares, fused AdamW, staging
    copy through a 1-rank communicator, including an offset slice that must not touch its neighbours)."""
    import torch
    from .ops.optim import adamw_reference, fused_adamw_, scratch_floats, sum_squares_
    dev = torch.device("cuda", 0)
    x = torch.randn(4096, device=dev).to(torch.bfloat16)
    out = torch.zeros(1, device=dev)
    sum_squares_(x, out, torch.zeros(scratch_floats(4096), device=dev))
    ok = torch.allclose(out[0], x.float().pow(2).sum(), rtol=1e-5)
    comm = Communicator(1, get_unique_id(), 0, transport="cuda")
    buf = torch.zeros(4096, device=dev)
    src = torch.arange(1024, device=dev, dtype=torch.float32)
    comm.all_reduce(src, buf[1024:2048])
    torch.cuda.synchronize()
    ok = ok and torch.equal(buf[1024:2048], src) and buf[:1024].abs().sum() == 0 and buf[2048:].abs().sum() == 0
    comm.destroy()
    print(f"kernels: {'ok' if ok else 'FAIL'}")
    return 0 if ok else 1


def probe_comm(a) -> int:
    comm = _comm(a.transport)
    if comm.rank == 0:
        print(comm.topo_xml())
    for coll, nbytes in (("allreduce", 1 << 10), ("allreduce", 1 << 20), ("allreduce", 1 << 30), ("allgather", 1 << 20)):
        print(f"rank {comm.rank}/{comm.size} transport {comm.transport} nvls {comm.nvls}: {coll} {nbytes} B -> {comm.pick_algo(coll, nbytes)}")
    comm.finalize(); comm.destroy()
    return 0


def probe_coll(a) -> int:
    comm = _comm(a.transport)
    n, r, cnt = comm.size, comm.rank, a.count
    cuda = comm.transport == "cuda"
    if cuda:
        import torch
        mk = lambda v: torch.tensor(np.asarray(v, dtype=np.float32), device="cuda")
        back = lambda t: t.cpu().numpy()
    else:
        mk = lambda v: np.asarray(v, dtype=np.float32).copy()
        back = lambda t: t
    ok = True
    if a.op == "allreduce":
        x = mk(np.full(cnt, r + 1.0)); comm.all_reduce(x)
        ok = np.all(back(x) == n * (n + 1) / 2)
    elif a.op == "allgather":
        out = mk(np.zeros(cnt * n)); comm.all_gather(mk(np.full(cnt, float(r))), out)
        ok = np.array_equal(back(out), np.repeat(np.arange(n, dtype=np.float32), cnt))
    elif a.op == "reducescatter":
        out = mk(np.zeros(cnt)); comm.reduce_scatter(mk(np.repeat(np.arange(n, dtype=np.float32), cnt)), out)
        ok = np.all(back(out) == r * n)
    elif a.op == "broadcast":
        x = mk(np.full(cnt, 42.0 if r == a.root else 0.0)); comm.broadcast(x if r == a.root else None, x, root=a.root)
        ok = np.all(back(x) == 42.0)
    elif a.op == "reduce":
        out = mk(np.zeros(cnt)); comm.reduce(mk(np.full(cnt, r + 1.0)), out if r == a.root else None, root=a.root)
        ok = r != a.root or np.all(back(out) == n * (n + 1) / 2)
    elif a.op == "alltoall":
        s = mk(np.repeat(r * n + np.arange(n, dtype=np.float32), cnt)); out = mk(np.zeros(cnt * n))
        comm.all_to_all(s, out)
        ok = np.array_equal(back(out), np.repeat(np.arange(n, dtype=np.float32) * n + r, cnt))     # provenance tag src*n+dst
    if cuda:
        import torch
        torch.cuda.synchronize()
    print(f"rank {r}: {a.op} count {cnt} algo {comm.last_algo}: {'ok' if ok else 'FAIL'}")
    comm.finalize(); comm.destroy()
    return 0 if ok else 1


def probe_bootstrap(a) -> int:
    """Every rank contributes 1000 + rank through the control plane and checks the gathered table
    (src/bootstrap.cc:88-109 of the reference)."""
    import struct
    comm = _comm("tcp")
    got = [struct.unpack("i", b)[0] for b in comm.host_all_gather(struct.pack("i", 1000 + comm.rank))]
    ok = got == [1000 + r for r in range(comm.size)]
    print(f"rank {comm.rank}: bootstrap all-gather {got}: {'ok' if ok else 'FAIL'}")
    comm.finalize(); comm.destroy()
    return 0 if ok else 1


def probe_m2m(a) -> int:
    """Rank 0 sends `--bytes` bytes of the pattern data[i] = i & 0xff to rank 1 over the striped TCP transport
    and rank 1 verifies every byte (src/transport/m2m.cc:372-404 of the reference); other ranks idle."""
    import time
    comm = _comm("tcp")
    ok, n = True, a.bytes
    if comm.size < 2:
        print("m2m: needs two ranks")
        comm.destroy()
        return 1
    pattern = (np.arange(n, dtype=np.uint64) & 0xff).astype(np.uint8)
    if comm.rank == 0:
        comm.send(pattern[:64], 1)                         # opens the connection
        comm.host_barrier()
        t0 = time.perf_counter()
        comm.send(pattern, 1)
        print(f"rank 0: sent {n} bytes in {(time.perf_counter() - t0) * 1e3:.2f} ms")
    elif comm.rank == 1:
        data = np.zeros(n, dtype=np.uint8)
        comm.recv(data[:64], 0)
        comm.host_barrier()
        t0 = time.perf_counter()
        comm.recv(data, 0)
        dt = time.perf_counter() - t0
        ok = bool(np.array_equal(data, pattern))
        print(f"rank 1: received {n} bytes in {dt * 1e3:.2f} ms ({n / dt / 1e9:.2f} GB/s): {'ok' if ok else 'FAIL'}")
    else:
        comm.host_barrier()
    comm.finalize(); comm.destroy()
    return 0 if ok else 1


def probe_discover(a) -> int:
    """Prints what discovery and the planner agreed on (src/graph/discover.cc:178-221 of the reference): one line
    per rank and link of the topology, the multicast capability and each algorithm's plan."""
    import xml.etree.ElementTree as ET
    comm = _comm(a.transport)
    root = ET.fromstring(comm.topo_xml())
    if comm.rank == 0:
        for el in root.iter():
            if el.tag != root.tag and el.attrib:
                print(f"{el.tag}: " + " ".join(f"{k}={v}" for k, v in el.attrib.items()))
    print(f"rank {comm.rank}/{comm.size}: transport {comm.transport}, nvls {comm.nvls}")
    ok = sum(1 for el in root.iter() if el.tag in ("gpu", "node", "rank")) >= 1 or len(list(root)) > 0
    comm.finalize(); comm.destroy()
    return 0 if ok else 1


def probe_bw(a) -> int:
    os.environ["MCCL_CALIBRATE"] = "1"
    comm = _comm("cuda")
    if comm.rank == 0:
        print(comm.topo_xml())
    comm.finalize(); comm.destroy()
    return 0


def main() -> int:
    ap = argparse.ArgumentParser(prog="python -m mccl_b200.probe")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("alloc"); p.add_argument("--size", type=int, default=65536); p.add_argument("--count", type=int, default=4)
    p = sub.add_parser("trees"); p.add_argument("--max", type=int, default=256)
    p = sub.add_parser("connect"); p.add_argument("--nodes", type=int, default=16); p.add_argument("--cuda", action="store_true")
    p = sub.add_parser("xml"); p.add_argument("--nodes", type=int, default=8); p.add_argument("--cuda", action="store_true"); p.add_argument("--out", default="")
    sub.add_parser("gpu")
    sub.add_parser("kernels")
    p = sub.add_parser("comm"); p.add_argument("--transport", default=None)
    p = sub.add_parser("coll"); p.add_argument("--op", default="allreduce"); p.add_argument("--count", type=int, default=1 << 16)
    p.add_argument("--root", type=int, default=0); p.add_argument("--transport", default=None)
    p = sub.add_parser("bw"); p.add_argument("--mbytes", type=int, default=256)
    sub.add_parser("bootstrap")
    p = sub.add_parser("m2m"); p.add_argument("--bytes", type=int, default=8 << 20)
    p = sub.add_parser("discover"); p.add_argument("--transport", default=None)
    a = ap.parse_args()
    return globals()["probe_" + a.cmd](a)


if __name__ == "__main__":
    sys.exit(main())
