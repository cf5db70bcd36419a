"""Single-process unit tests of the host-side subsystems on synthetic inputs (the role of the reference's
MCCL_TREES_MAIN, MCCL_CONNECT_MAIN, MCCL_XML_MAIN and MCCL_ALLOC_MAIN probes)."""
import ctypes as C
import os

import numpy as np
import pytest

import mccl_b200 as mccl
from mccl_b200 import _lib as L


def test_version_and_strings(lib):
    v = C.c_int()
    assert lib.mcclGetVersion(C.byref(v)) == 0 and v.value == 100
    assert lib.mcclResultStr(L.REMOTE_ERROR) == b"remote error"
    assert lib.mcclDataTypeStr(L.BFLOAT16) == b"bfloat16"
    assert lib.mcclRedOpStr(L.AVG) == b"avg"
    assert [lib.mcclAlgoStr(i) for i in range(5)] == [b"ring", b"tree", b"oneshot", b"twoshot", b"nvls"]
    assert [lib.mcclDataSize(i) for i in range(10)] == [1, 1, 4, 4, 8, 8, 2, 2, 4, 8]
    assert lib.mcclDataSize(42) == 0


def test_param_parsing(lib, monkeypatch):
    monkeypatch.setenv("MCCL_UNIT_X", "0x20")
    assert lib.mcclDbgParam(b"MCCL_UNIT_X", 5) == 32
    monkeypatch.setenv("MCCL_UNIT_X", "junk")
    assert lib.mcclDbgParam(b"MCCL_UNIT_X", 5) == 5
    monkeypatch.delenv("MCCL_UNIT_X")
    assert lib.mcclDbgParam(b"MCCL_UNIT_X", -7) == -7


def test_algo_list_parsing(lib):
    en = (C.c_int * 5)()
    assert lib.mcclDbgParseList(b"ring,tree", en) == 0 and list(en) == [1, 1, 0, 0, 0]
    assert lib.mcclDbgParseList(b"^ring", en) == 0 and list(en) == [0, 1, 1, 1, 1]
    assert lib.mcclDbgParseList(b"NVLS", en) == 0 and list(en) == [0, 0, 0, 0, 1]
    assert lib.mcclDbgParseList(b"", en) == 0 and list(en) == [1] * 5
    assert lib.mcclDbgParseList(b"bogus", en) == L.INVALID_ARGUMENT


NP_TYPES = {L.INT8: np.int8, L.UINT8: np.uint8, L.INT32: np.int32, L.UINT32: np.uint32, L.INT64: np.int64,
            L.UINT64: np.uint64, L.FLOAT16: np.float16, L.FLOAT32: np.float32, L.FLOAT64: np.float64}


@pytest.mark.parametrize("dt", sorted(NP_TYPES))
@pytest.mark.parametrize("op", ["sum", "prod", "max", "min"])
def test_host_reduce_all_types(lib, dt, op):
    npdt = NP_TYPES[dt]
    rng = np.random.default_rng(dt * 7 + len(op))
    n = 4099 if dt != L.FLOAT32 else (1 << 21) + 3      # the large one takes the parallel path
    if np.dtype(npdt).kind == "f":
        a, b = rng.uniform(-2, 2, n).astype(npdt), rng.uniform(-2, 2, n).astype(npdt)
    else:
        a, b = rng.integers(0, 11, n).astype(npdt), rng.integers(0, 11, n).astype(npdt)
    ref = {"sum": a + b, "prod": a * b, "max": np.maximum(a, b), "min": np.minimum(a, b)}[op]
    dst = a.copy()
    assert lib.mcclDbgHostReduce(dst.ctypes.data, b.ctypes.data, n, dt, L.OPS[op]) == 0
    if npdt == np.float16:
        assert np.allclose(dst.astype(np.float32), ref.astype(np.float32), rtol=2e-3, atol=2e-3)
    else:
        assert np.array_equal(dst, ref)


def test_host_reduce_bf16_and_scale(lib):
    import torch
    a = torch.randn(5001).to(torch.bfloat16)
    b = torch.randn(5001).to(torch.bfloat16)
    dst = a.clone()
    assert lib.mcclDbgHostReduce(dst.data_ptr(), b.data_ptr(), 5001, L.BFLOAT16, L.SUM) == 0
    assert torch.equal(dst, (a.float() + b.float()).to(torch.bfloat16))       # widen, add, round to nearest even
    nan = torch.tensor([float("nan"), 1.0]).to(torch.bfloat16)
    one = torch.ones(2).to(torch.bfloat16)
    lib.mcclDbgHostReduce(nan.data_ptr(), one.data_ptr(), 2, L.BFLOAT16, L.SUM)
    assert torch.isnan(nan[0]) and nan[1] == 2
    x = np.arange(-8, 8, dtype=np.int32)
    y = x.copy()
    assert lib.mcclDbgHostScale(y.ctypes.data, y.size, L.INT32, 3) == 0
    assert np.array_equal(y, np.trunc(x / 3).astype(np.int32))               # integer avg truncates
    f = np.linspace(-1, 1, 1001, dtype=np.float32)
    g = f.copy()
    lib.mcclDbgHostScale(g.ctypes.data, g.size, L.FLOAT32, 4)
    assert np.allclose(g, f / 4)


def _dtree(lib, n, r):
    out = (C.c_int * 6)()
    lib.mcclDbgDtree(n, r, out)
    return list(out)


@pytest.mark.parametrize("n", list(range(1, 66)) + [100, 127, 128, 129, 255, 256])
def test_double_binary_tree_invariants(lib, n):
    trees = [_dtree(lib, n, r) for r in range(n)]
    for t in (0, 1):
        ups = [trees[r][3 * t] for r in range(n)]
        kids = [[c for c in trees[r][3 * t + 1:3 * t + 3] if c >= 0] for r in range(n)]
        roots = [r for r in range(n) if ups[r] < 0]
        assert len(roots) == 1
        for r in range(n):
            for c in kids[r]:
                assert 0 <= c < n and ups[c] == r                       # parent/child agree
            if ups[r] >= 0:
                assert r in kids[ups[r]]
        seen, stack = set(), [roots[0]]                                  # every rank reachable from the root
        while stack:
            v = stack.pop()
            assert v not in seen
            seen.add(v)
            stack.extend(kids[v])
        assert seen == set(range(n))
    if n > 2:
        leaf0 = {r for r in range(n) if trees[r][1] < 0 and trees[r][2] < 0}
        leaf1 = {r for r in range(n) if trees[r][4] < 0 and trees[r][5] < 0}
        assert not (leaf0 & leaf1)                                       # nobody is a leaf in both trees
        r0 = [r for r in range(n) if trees[r][0] < 0][0]
        r1 = [r for r in range(n) if trees[r][3] < 0][0]
        assert r0 != r1


def _channel(lib, n, r, cuda, dtree=0, cap=8):
    out = (C.c_int * (4 + 2 * (2 + cap)))()
    assert lib.mcclDbgSyntheticChannel(n, r, cuda, dtree, out, cap) == 0
    v = list(out)
    a, b = v[4:6 + cap], v[6 + cap:]
    return {"prev": v[0], "next": v[1], "flat": v[2], "dtree": v[3], "upA": a[0], "downA": [c for c in a[2:2 + a[1]]],
            "upB": b[0], "downB": [c for c in b[2:2 + b[1]]]}


@pytest.mark.parametrize("n,cuda", [(2, 0), (4, 0), (16, 0), (2, 1), (8, 1), (5, 1)])
def test_channel_connect(lib, n, cuda):
    chans = [_channel(lib, n, r, cuda, cap=16) for r in range(n)]
    for r, ch in enumerate(chans):                                       # ring: rank order, mutual neighbours
        assert ch["next"] == (r + 1) % n and ch["prev"] == (r - 1) % n
    roots = [r for r in range(n) if chans[r]["upA"] < 0]
    assert len(roots) == 1
    for r, ch in enumerate(chans):
        for c in ch["downA"]:
            assert chans[c]["upA"] == r
    if cuda and n > 2:
        assert all(ch["dtree"] for ch in chans)                          # NVSwitch: every pair has its own path
    if not cuda and n <= 8:
        assert all(ch["flat"] for ch in chans)                           # uniform LAN: depth-1 star
        assert sum(len(ch["downA"]) for ch in chans) == n - 1
    if not cuda and n > 8:
        assert all(ch["dtree"] for ch in chans)                          # above MCCL_DTREE_MIN_RANKS


def test_forced_dtree_on_tcp(lib):
    chans = [_channel(lib, 6, r, 0, dtree=1) for r in range(6)]
    assert all(ch["dtree"] for ch in chans)
    assert len([1 for ch in chans if ch["upB"] < 0]) == 1


def _xml(lib, n, cuda, bw=0.0, nvls=0):
    p = C.c_void_p()
    assert lib.mcclDbgSyntheticTopoXml(n, cuda, C.c_float(bw), nvls, C.byref(p)) == 0
    s = C.string_at(p).decode()
    lib.mcclFreeString(p)
    return s


def test_topology_xml_and_round_trip(lib):
    import xml.etree.ElementTree as ET
    s = _xml(lib, 8, 1, 0.0, 1)
    root = ET.fromstring(s)
    assert root.tag == "system" and root.get("ranks") == "8" and root.get("nvls") == "1"
    gpus = root.findall("gpu")
    assert len(gpus) == 8 and all(len(g.findall("link")) == 7 for g in gpus)
    assert all(l.get("type") == "NVL" and float(l.get("bw")) == 900.0 for g in gpus for l in g.findall("link"))
    algos = {a.get("name"): a for a in root.findall("algo")}
    assert set(algos) == {"ring", "tree", "oneshot", "twoshot", "nvls"} and all(a.get("viable") == "1" for a in algos.values())
    out = C.c_void_p()
    assert lib.mcclDbgXmlRoundTrip(s.encode(), C.byref(out)) == 0
    again = C.string_at(out).decode()
    lib.mcclFreeString(out)
    assert ET.tostring(ET.fromstring(again)) == ET.tostring(root)
    tcp = ET.fromstring(_xml(lib, 3, 0, 2.5))
    assert len(tcp.findall("host")) == 3
    assert {a.get("name"): a.get("viable") for a in tcp.findall("algo")}["nvls"] == "0"
    assert all(float(l.get("bw")) == 2.5 for h in tcp.findall("host") for l in h.findall("link"))


def test_paths_detect_missing_peer_link(lib):
    n = 4
    types = (C.c_int * (n * n))()
    hops = (C.c_int * (n * n))()
    types[0] = 2                                   # sever NVLink between GPUs 1 and 2
    assert lib.mcclDbgPaths(n, 1, types, hops) == 0
    t = np.array(list(types)).reshape(n, n)
    h = np.array(list(hops)).reshape(n, n)
    assert t[0, 0] == 0 and h[0, 0] == 0                                 # LOC
    assert t[0, 1] == 1 and h[0, 1] == 1                                 # one NVLink hop
    assert t[1, 2] == 2 and h[1, 2] == 2                                 # relayed over another GPU
    assert t[2, 1] == 2


def _pick(lib, n, cuda, nvls, nbytes, coll="allreduce", dt=L.FLOAT32, op=L.SUM, algos=b""):
    a = C.c_int()
    times = (C.c_float * 5)()
    rc = lib.mcclDbgTunerPick(n, cuda, nvls, nbytes, L.COLLS[coll], dt | (op << 8), algos, C.byref(a), times)
    assert rc == 0
    return L.ALGO_NAMES[a.value], list(times)


def test_tuner_choices(lib):
    assert _pick(lib, 8, 1, 1, 4096)[0] == "oneshot"                     # latency bound
    assert _pick(lib, 8, 1, 1, 1 << 30)[0] == "nvls"                     # the switch reduces: least traffic
    assert _pick(lib, 8, 1, 0, 1 << 30)[0] == "twoshot"
    assert _pick(lib, 8, 1, 1, 1 << 30, op=L.PROD)[0] == "twoshot"       # multimem has no product
    assert _pick(lib, 8, 1, 1, 1 << 30, algos=b"ring,tree")[0] == "ring"
    assert _pick(lib, 8, 1, 1, 1 << 30, algos=b"^nvls,twoshot")[0] in ("ring", "tree")
    name, t = _pick(lib, 8, 1, 1, 1 << 30)
    assert t[L.ALGO_NVLS] < t[L.ALGO_TWOSHOT] < t[L.ALGO_RING] < t[L.ALGO_TREE] < t[L.ALGO_ONESHOT]
    assert _pick(lib, 4, 0, 0, 1 << 10)[0] == "oneshot"                  # tcp: direct path below 2 MiB
    assert _pick(lib, 4, 0, 0, 64 << 20)[0] == "ring"
    assert _pick(lib, 4, 0, 0, 1 << 10, coll="broadcast")[0] in ("ring", "tree")
    # cuda without NVLS: ring and tree can run every collective but are never the model's choice; forced, they are used
    for coll in ("allgather", "reducescatter", "broadcast", "reduce"):
        for nbytes in (1 << 10, 1 << 20, 1 << 30):
            assert _pick(lib, 8, 1, 0, nbytes, coll=coll)[0] in ("oneshot", "twoshot")
            assert _pick(lib, 8, 1, 1, nbytes, coll=coll)[0] == "nvls"
        assert _pick(lib, 8, 1, 1, 1 << 20, coll=coll, algos=b"ring")[0] == "ring"
        assert _pick(lib, 8, 1, 1, 1 << 20, coll=coll, algos=b"tree")[0] == "tree"


def test_mem_pool(lib):
    pool = C.c_void_p()
    assert lib.mcclMemPoolCreate(1 << 16, 2, C.byref(pool)) == 0
    bufs = [L.Buf() for _ in range(3)]
    for b in bufs:
        assert lib.mcclMemPoolAlloc(pool, C.byref(b)) == 0               # third allocation grows the pool
        assert b.host % os.sysconf("SC_PAGESIZE") == 0 and b.size == 1 << 16
    assert len({b.host for b in bufs}) == 3
    total, free = C.c_int(), C.c_int()
    lib.mcclMemPoolStats(pool, C.byref(total), C.byref(free))
    assert (total.value, free.value) == (3, 0)
    assert lib.mcclMemPoolFree(pool, C.byref(bufs[1])) == 0
    assert lib.mcclMemPoolFree(pool, C.byref(bufs[1])) == L.INVALID_USAGE  # double free
    again = L.Buf()
    assert lib.mcclMemPoolAlloc(pool, C.byref(again)) == 0 and again.host == bufs[1].host   # reuse
    assert lib.mcclMemPoolDestroy(pool) == 0


def test_single_rank_tcp_comm():
    comm = mccl.Communicator(1, mccl.get_unique_id(), 0, transport="tcp")
    x = np.arange(10, dtype=np.float32)
    y = np.zeros_like(x)
    comm.all_reduce(x, y, op="avg")
    assert np.array_equal(x, y)
    comm.all_gather(x, y)
    assert np.array_equal(x, y)
    assert comm.transport == "tcp" and comm.size == 1 and not comm.nvls
    assert "<system" in comm.topo_xml()
    comm.finalize(); comm.destroy()


def test_unknown_transport_is_refused():
    with pytest.raises(mccl.MCCLError) as e:
        mccl.Communicator(1, mccl.get_unique_id(), 0, transport="carrier-pigeon")
    assert e.value.code == L.INVALID_ARGUMENT


def test_unique_ids_differ():
    a, b = mccl.get_unique_id(), mccl.get_unique_id()
    assert a != b


def test_trace_file_is_chrome_json(tmp_path):
    import json
    import subprocess
    import sys
    code = ("import numpy as np, mccl_b200 as m\n"
            "c = m.Communicator(1, m.get_unique_id(), 0, transport='tcp')\n"
            "x = np.ones(64, np.float32)\n"
            "c.all_reduce(x); c.all_gather(x, x.copy()); c.finalize(); c.destroy()\n")
    env = dict(os.environ, MCCL_TRACE=str(tmp_path / "trace"), PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    subprocess.run([sys.executable, "-c", code], env=env, check=True)
    data = json.load(open(tmp_path / "trace.0.json"))
    names = [e["name"] for e in data["traceEvents"]]
    assert names == ["AllReduce", "AllGather"]
    assert all(e["ph"] == "X" and e["dur"] >= 0 and e["args"]["bytes"] > 0 for e in data["traceEvents"])


def test_env_knobs_at_init(tmp_path, monkeypatch):
    """MCCL_TOPO_DUMP_FILE, MCCL_ALGO and MCCL_TUNER_CACHE are read when a communicator is created."""
    import subprocess
    import sys
    import xml.etree.ElementTree as ET
    cache = tmp_path / "tuner.txt"
    cache.write_text("ring 7.5 2.5 3.25\ntree 1 1 1\n")
    code = ("import mccl_b200 as m\n"
            "c = m.Communicator(1, m.get_unique_id(), 0, transport='tcp')\n"
            "print('PICK', c.pick_algo('allreduce', 1 << 26))\n"
            "c.destroy()\n")
    env = dict(os.environ, MCCL_TOPO_DUMP_FILE=str(tmp_path / "topo.xml"), MCCL_ALGO="^ring", MCCL_TUNER_CACHE=str(cache),
               PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    out = subprocess.run([sys.executable, "-c", code], env=env, check=True, capture_output=True, text=True).stdout
    assert "PICK tree" in out                                  # ring is denied
    root = ET.parse(tmp_path / "topo.xml").getroot()
    ring = [a for a in root.findall("algo") if a.get("name") == "ring"][0]
    assert float(ring.get("alpha_us")) == 7.5 and float(ring.get("step_us")) == 2.5 and float(ring.get("model_bw")) == 3.25


def test_work_split_covers_every_unit_once(lib):
    """The CTA work split of the collective kernels: tiles of all CTAs partition [0, V) for any size and CTA count."""
    f = lib.mcclDbgWorkSplit
    f.restype = C.c_int
    f.argtypes = [C.c_uint64, C.c_int, C.c_int, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.c_int]
    cap = 4096
    lo, hi = (C.c_uint64 * cap)(), (C.c_uint64 * cap)()
    for V in (0, 1, 7, 511, 512, 513, 16384, 16385, 1_000_003, 32 * 16384, 32 * 16384 + 5, 50_000_000):
        for G in (1, 2, 3, 16, 32, 64, 128):
            spans = []
            for cta in range(G):
                k = f(V, G, cta, lo, hi, cap)
                assert k <= cap
                spans += [(lo[i], hi[i]) for i in range(k)]
            spans.sort()
            pos = 0
            for a, b in spans:
                assert a == pos and b > a, (V, G, a, b, pos)
                pos = b
            assert pos == V, (V, G, pos)


def test_shards_are_16_byte_aligned_and_cover_the_message(lib):
    f = lib.mcclDbgShard
    f.restype = None
    f.argtypes = [C.c_uint64, C.c_int, C.c_int, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    for nbytes in (1, 15, 16, 17, 100, 4099, 1 << 20, (1 << 30) + 6, 34359738368):
        for n in (2, 3, 4, 8, 16):
            pos = 0
            for r in range(n):
                off, end = C.c_uint64(), C.c_uint64()
                f(nbytes, n, r, C.byref(off), C.byref(end))
                assert off.value == pos and off.value % 16 == 0 and end.value >= off.value
                pos = end.value
            assert pos == nbytes                                # the last shard takes the tail


def test_gemm_tile_order_visits_every_tile_once(lib):
    """Rasterisation of the tcgen05 GEMM: plain, all-gather (own shard first) and reduce-scatter (own block last)."""
    f = lib.mcclDbgGemmTile
    f.restype = C.c_int
    f.argtypes = [C.c_int] * 7 + [C.POINTER(C.c_int)] * 4
    for mode, M, N, n in ((0, 8192, 3584, 1), (0, 384, 448, 1), (0, 128 * 13, 64, 1), (1, 8192, 3584, 8), (2, 8192, 8192, 8),
                          (1, 8192, 7168, 4), (2, 2048, 1024, 2), (2, 128 * 6, 192, 3)):
        for rank in range(n):
            s_, nt_, bn, panel = C.c_int(), C.c_int(), C.c_int(), C.c_int()
            total = f(mode, M, N, n, rank, 148, 0, C.byref(s_), C.byref(nt_), C.byref(bn), C.byref(panel))
            assert total == (M // 128) * (N // bn.value) and N % bn.value == 0
            seen, order = set(), []
            for t in range(total):
                assert f(mode, M, N, n, rank, 148, t, C.byref(s_), C.byref(nt_), C.byref(bn), C.byref(panel)) == total
                assert 0 <= s_.value < M // 128 and 0 <= nt_.value < N // bn.value
                seen.add((s_.value, nt_.value)); order.append(s_.value)
            assert len(seen) == total                               # a bijection
            per_block = (M // 128) // n
            blocks = [order[i] // per_block for i in range(0, total, per_block * (N // bn.value))]
            if mode == 1:
                assert blocks == [(rank + i) % n for i in range(n)]     # own shard first, then in arrival order
            if mode == 2:
                assert blocks == [(rank + 1 + i) % n for i in range(n)]  # peers' blocks first, own block last


def test_tuner_model_tracks_measured_times(lib):
    """The cost model's constants were fitted on 8 B200; these are times measured there (us, bf16 sum, forced
    algorithm).  A change of the constants that moves a prediction by more than 35 % should be a deliberate one."""
    measured = {  # algorithm -> {bytes: us}
        "nvls":    {1 << 20: 32.7, 4 << 20: 38.8, 16 << 20: 71.4, 64 << 20: 173.4, 256 << 20: 585.8},
        "twoshot": {1 << 10: 55.0, 256 << 20: 761.0},
        "oneshot": {1 << 10: 26.0, 1 << 20: 76.0},
        "ring":    {1 << 10: 148.0, 256 << 20: 2292.0},
        "tree":    {1 << 10: 94.0, 256 << 20: 12477.0},
    }
    for algo, cells in measured.items():
        for nbytes, us in cells.items():
            _, times = _pick(lib, 8, 1, 1, nbytes, dt=L.BFLOAT16)
            model = times[L.ALGOS[algo]]
            assert 0.65 * us <= model <= 1.35 * us, (algo, nbytes, model, us)


def test_fused_mlp_backward_formulas_on_cpu():
    """The hand-written backward of FusedTensorParallelMLP (recomputed pre-activation, SiLU derivative, weight and input
    gradients) against autograd, with the fused forward kernels replaced by their plain PyTorch meaning."""
    import torch
    from mccl_b200.parallel.tp import _FusedMLPFunction
    comm = mccl.Communicator(1, mccl.get_unique_id(), 0, transport="tcp")

    class FakeLayer:                      # what TensorParallelFFN.forward computes, without the kernels
        def __init__(self, w_up, w_down):
            self.comm, self.w_up, self.w_down, self.x_full = comm, w_up, w_down, None

        def forward(self, x):
            self.x_full = x.detach().clone()
            return torch.nn.functional.silu(self.x_full @ self.w_up.t()) @ self.w_down.t()

    torch.manual_seed(0)
    x = torch.randn(12, 8, dtype=torch.float64, requires_grad=True)
    w_up = torch.randn(20, 8, dtype=torch.float64, requires_grad=True)
    w_down = torch.randn(8, 20, dtype=torch.float64, requires_grad=True)
    tgt = torch.randn(12, 8, dtype=torch.float64)
    y = _FusedMLPFunction.apply(x, w_up, w_down, FakeLayer(w_up.detach(), w_down.detach()))
    (y * tgt).sum().backward()
    got = [t.grad.clone() for t in (x, w_up, w_down)]
    for t in (x, w_up, w_down):
        t.grad = None
    ref = torch.nn.functional.silu(x @ w_up.t()) @ w_down.t()
    (ref * tgt).sum().backward()
    assert torch.allclose(y, ref.detach(), atol=1e-12)
    for g, t in zip(got, (x, w_up, w_down)):
        assert torch.allclose(g, t.grad, atol=1e-5, rtol=1e-5), (g - t.grad).abs().max().item()
    comm.destroy()


def test_moe_dispatch_combine_autograd_on_cpu(monkeypatch):
    """The autograd wiring of the fused dispatch / combine (a dispatch's backward is a gather of the slot gradients, a
    combine's backward scatters gate * dy and gives the gate <dy, row>) with the two kernels replaced by one-rank
    PyTorch stand-ins of what they do."""
    import torch
    from mccl_b200.ops import moe as M

    class Buf:
        def __init__(self, e, c, d):
            self.e, self.c, self.d = e, c, d
            self.data = torch.zeros(1, e, c, d, dtype=torch.float64)

    def scatter(buf, x, flat, scale):
        buf.data.zero_()
        keep = flat >= 0
        rows = x[keep] if scale is None else x[keep] * scale[keep].unsqueeze(-1).to(x.dtype)
        buf.data.view(-1, buf.d)[flat[keep].long()] = rows

    def gather(buf, flat, scale, n_tokens):
        out = torch.zeros(n_tokens, buf.d, dtype=buf.data.dtype)
        keep = flat >= 0
        rows = buf.data.view(-1, buf.d)[flat[keep].long()]
        out[keep] = rows if scale is None else rows * scale[keep].unsqueeze(-1).to(rows.dtype)
        return out

    monkeypatch.setattr(M, "_scatter", scatter)
    monkeypatch.setattr(M, "_gather", gather)
    torch.manual_seed(0)
    e, c, d, T = 3, 2, 5, 9
    flat = torch.tensor([0, 2, -1, 3, 5, -1, 1, 4, -1], dtype=torch.int32)          # three dropped tokens
    x = torch.randn(T, d, dtype=torch.float64, requires_grad=True)
    gate = torch.rand(T, dtype=torch.float64, requires_grad=True)
    w = torch.randn(d, d, dtype=torch.float64, requires_grad=True)                   # a stand-in "expert"
    tgt = torch.randn(T, d, dtype=torch.float64)
    buf, gbuf = Buf(e, c, d), Buf(e, c, d)
    recv = M.dispatch(x, flat, buf, gbuf)
    y = M.combine(recv @ w, flat, gate, buf, gbuf)
    (y * tgt).sum().backward()
    got = [t.grad.clone() for t in (x, gate, w)]
    for t in (x, gate, w):
        t.grad = None
    keep = flat >= 0
    ref = torch.zeros(T, d, dtype=torch.float64)
    ref[keep] = (x[keep] @ w) * gate[keep].float().double().unsqueeze(-1)
    (ref * tgt).sum().backward()
    assert torch.allclose(y, ref.detach(), atol=1e-6)
    for g, t, name in zip(got, (x, gate, w), ("dx", "dgate", "dw")):
        assert torch.allclose(g, t.grad, atol=1e-5, rtol=1e-5), (name, (g - t.grad).abs().max().item())


def test_result_fatal_matches_the_latching_rule(lib):
    """System, internal and remote errors latch on a communicator (src/include/comm.h:106-108 of the reference); usage
    errors and mcclInProgress do not."""
    fatal = {L.SYSTEM_ERROR, L.INTERNAL_ERROR, L.REMOTE_ERROR}
    for code in range(8):
        assert bool(lib.mcclResultFatal(code)) == (code in fatal)


def test_python_wrappers_refuse_mismatched_buffers():
    """Sizes, dtypes and devices are checked in Python: a short receive buffer must raise, not be overrun."""
    import numpy as np
    import torch
    import mccl_b200 as mccl
    comm = mccl.Communicator(1, mccl.get_unique_id(), 0, transport="tcp")
    x = torch.ones(16)
    with pytest.raises(ValueError):
        comm.all_reduce(x, torch.empty(15))
    with pytest.raises(ValueError):
        comm.all_reduce(x, torch.empty(16, dtype=torch.float64))
    with pytest.raises(TypeError):
        comm.all_reduce(x, np.empty(16, dtype=np.float32))
    with pytest.raises(ValueError):
        comm.all_gather(x, torch.empty(15))
    with pytest.raises(ValueError):
        comm.reduce_scatter(torch.ones(7), torch.empty(8))
    with pytest.raises(ValueError):
        comm.broadcast(torch.ones(7), torch.empty(8))
    with pytest.raises(ValueError):
        comm.reduce(x, torch.empty(8))
    with pytest.raises(ValueError):
        comm.all_to_all(x, torch.empty(8))
    with pytest.raises(ValueError):
        comm.gather(x, torch.empty(8))
    with pytest.raises(ValueError):
        comm.scatter(torch.ones(4), torch.empty(8))
    with pytest.raises(ValueError):
        comm.all_to_all_v(x, [17], torch.empty(32), [17])
    # well-formed calls still go through
    y = torch.empty(16)
    comm.all_reduce(x, y)
    comm.all_gather(x, y)
    comm.broadcast(x, y)
    assert torch.equal(x, y)
    comm.finalize(); comm.destroy()


def test_symmetric_pool_bookkeeping():
    """One allocation, local first-fit sub-allocations: aligned, disjoint, merged on free, refused when full."""
    import torch
    import mccl_b200 as mccl
    comm = mccl.Communicator(1, mccl.get_unique_id(), 0, transport="tcp")
    pool = comm.pool(64 * 1024)
    a = pool.empty(1000, torch.float32)           # 4000 bytes -> 4096
    b = pool.empty(3, torch.bfloat16)             # 16 bytes minimum -> 256
    c = pool.empty((8, 16), torch.float32)
    assert a.data_ptr() % 256 == 0 and b.data_ptr() == a.data_ptr() + 4096 and c.data_ptr() == b.data_ptr() + 256
    a.fill_(1.0); b.fill_(2.0); c.fill_(3.0)
    assert a.sum() == 1000 and c.shape == (8, 16) and float(b[0]) == 2.0
    st = pool.stats()
    assert st["total"] == 65536 and st["in_use"] == 4096 + 256 + 512
    pool.free(b)
    d = pool.empty(40, torch.float32)             # 160 bytes: first fit reuses b's range
    assert d.data_ptr() == a.data_ptr() + 4096
    pool.free(a); pool.free(d); pool.free(c)
    st = pool.stats()
    assert st["in_use"] == 0 and st["largest_free"] == 65536       # neighbours merged back into one range
    with pytest.raises(mccl.MCCLError):
        pool.empty(70000, torch.uint8)
    with pytest.raises(mccl.MCCLError):
        pool.free_raw(a.data_ptr())               # not live any more
    comm.all_reduce(pool.empty(16, torch.float32).zero_())      # a pool tensor is an ordinary buffer for the collectives
    pool.destroy()
    comm.finalize(); comm.destroy()


def test_build_resources_table_lists_every_kernel_family():
    """The report folded from the compiler's per-kernel output names the hot kernels and reports no spills in them."""
    from mccl_b200 import _build
    if not any(_build.OBJ.rglob("*.ptxas.txt")):
        pytest.skip("no compiler reports: the library was not built from source in this tree")
    table = _build.resources()
    rows = {line.split("|")[2].strip().strip("`"): [c.strip() for c in line.split("|")[1:-1]]
            for line in table.splitlines() if line.startswith("| ") and "`" in line}
    for kernel in ("gemm::tpGemm2Kernel", "nvlsKernel", "pullKernel", "oneShotKernel", "p2pKernel", "moeKernel", "adamwKernel"):
        assert kernel in rows, kernel
        assert rows[kernel][4] == "0", (kernel, rows[kernel])          # spill bytes


def test_send_recv_split_over_channels_tiles_every_message(lib):
    """Sender and receiver compute the cut of a message from (bytes, slot size, ranks) alone: the parts must tile
    the message exactly, every chunk must fit its channel's ring, and all CTAs of a full batch (one row of
    channels per direction and peer) must fit the 148 SMs at once, because they wait for one another across GPUs."""
    lib.mcclDbgP2pSplit.argtypes = [C.c_uint64, C.c_uint64, C.c_int, C.POINTER(C.c_uint64)]
    lib.mcclDbgP2pSplit.restype = None
    lib.mcclDbgP2pChannels.argtypes = [C.c_int]
    lib.mcclDbgP2pChannels.restype = C.c_int
    depth = 4
    rng = np.random.default_rng(7)
    for n in (2, 3, 4, 5, 8, 16):
        ch_max = lib.mcclDbgP2pChannels(n)
        assert 1 <= ch_max <= 32
        assert 2 * (n - 1) * ch_max <= 148
        default_slot = ch_max * depth * (512 << 10)
        for slot in (default_slot, 4096 << 10, 64 << 10, 16 << 10):
            sizes = [1, 13, 4096, 65536, 65537, (1 << 20) + 13, (5 << 20) + 4099, 256 << 20, (1 << 32) + 48]
            sizes += [int(x) for x in rng.integers(1, 1 << 28, size=40)]
            for nbytes in sizes:
                out = (C.c_uint64 * 3)()
                lib.mcclDbgP2pSplit(nbytes, slot, n, out)
                channels, per, chunk = int(out[0]), int(out[1]), int(out[2])
                assert 1 <= channels <= ch_max
                assert per % 256 == 0 and chunk % 16 == 0 and chunk >= 16
                assert channels * depth * chunk <= slot                      # every channel's ring lies inside the slot
                covered = 0
                for ch in range(channels):
                    lo = ch * per
                    if lo >= nbytes:
                        continue
                    covered += min(per, nbytes - lo)
                assert covered == nbytes, (n, slot, nbytes, channels, per)
                assert (channels - 1) * per < nbytes or channels == 1       # no channel starts beyond the end ...
                if nbytes >= channels * (64 << 10):
                    assert per >= 64 << 10                                   # ... and none carries a sliver of a large message


def test_collective_matrix_oracle_is_position_addressable_and_exact():
    """The checker of bench/coll_matrix.py: a window of a rank's input computed on its own equals the same slice of
    the whole input, the reference equals a plain reduction of all ranks' inputs, the windows cover start, middle and
    end, and the grading tells an exact result from a rounded one and from a wrong one."""
    import importlib.util
    import torch
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench", "coll_matrix.py")
    spec = importlib.util.spec_from_file_location("coll_matrix_under_test", path)
    cm = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(cm)
    dev = torch.device("cpu")
    n, world = 5000, 4
    for dname, dt in cm.DT.items():
        for op in ("sum", "prod", "max", "min", "avg"):
            whole = [cm.values(r, 0, n, dt, op, dev) for r in range(world)]
            assert whole[0].dtype == dt
            assert torch.equal(cm.values(2, 1234, 1300, dt, op, dev), whole[2][1234:1300])
            assert not torch.equal(whole[0], whole[1])                       # ranks differ
            ref = cm.reference(world, 100, 400, dt, op, dev)
            st = torch.stack([w[100:400].double() if dt.is_floating_point else w[100:400].long() for w in whole])
            if op == "sum":
                want = st.sum(0)
            elif op == "avg":
                want = st.sum(0) / world if dt.is_floating_point else torch.div(st.sum(0).to(dt), world, rounding_mode="trunc")
            elif op == "prod":
                want = st.prod(0)
            else:
                want = st.max(0).values if op == "max" else st.min(0).values
            assert torch.equal(ref.double(), want.double()), (dname, op)
    assert cm.windows(10) == [(0, 10)]
    big = 10 * cm.WINDOW + 3
    w = cm.windows(big)
    assert w[0] == (0, cm.WINDOW) and w[-1] == (big - cm.WINDOW, big) and w[1][0] % 8 == 0 and w[1][1] - w[1][0] == cm.WINDOW
    want = torch.tensor([1.0, 2.0, 3.0], dtype=torch.float64) / 3
    assert cm.grade(want.to(torch.bfloat16), want, torch.bfloat16) == "exact"
    assert cm.grade((want * (1 + 1e-2)).to(torch.bfloat16), want, torch.bfloat16) == "close"
    assert cm.grade((want + 1.0).to(torch.bfloat16), want, torch.bfloat16) == "WRONG"
    ints = torch.tensor([1, -2, 3], dtype=torch.int32)
    assert cm.grade(ints, ints.long(), torch.int32) == "exact" and cm.grade(ints + 1, ints.long(), torch.int32) == "WRONG"
