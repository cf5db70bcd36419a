"""GPU tests (marker `gpu`).  Single-GPU tests run the native kernels that need no peer; multi-GPU tests
start one process per GPU and compare every collective kernel with an fp64 / exact-integer PyTorch oracle."""
import os

import pytest
import torch

from _mp import assert_all_ok, run_ranks

pytestmark = pytest.mark.gpu

NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0
need2 = pytest.mark.skipif(NGPU < 2, reason="needs two GPUs")


def _require_cuda():
    if NGPU < 1:
        pytest.fail("GPU tests need a CUDA device (run the CPU tier with -m 'not gpu')")


def test_fused_adamw_matches_fp32_reference():
    _require_cuda()
    from mccl_b200.ops.optim import adamw_reference, fused_adamw_
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    for n in (8, 1000, 1003, (1 << 20) + 5):
        master = torch.randn(n, device=dev)
        param = master.to(torch.bfloat16)
        m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        rm, rma, rv = master.clone(), m.clone(), v.clone()
        for step in (1, 2, 3):
            grad = (torch.randn(n, device=dev) * 0.1).to(torch.bfloat16)
            g2 = grad.clone()
            fused_adamw_(param, master, m, v, grad, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, grad_scale=0.5, step=step)
            ref_p = adamw_reference(rm, rma, rv, g2, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, grad_scale=0.5, step=step)
            torch.cuda.synchronize()
            assert torch.allclose(master, rm, rtol=1e-5, atol=1e-6)
            assert torch.allclose(m, rma, rtol=1e-5, atol=1e-7) and torch.allclose(v, rv, rtol=1e-5, atol=1e-9)
            assert torch.equal(param, ref_p) or (param.float() - ref_p.float()).abs().max() <= 2 ** -7 * ref_p.float().abs().max()
            assert torch.count_nonzero(grad) == 0              # the kernel clears the gradient for the next step


def test_single_rank_cuda_communicator():
    _require_cuda()
    import mccl_b200 as mccl
    torch.cuda.set_device(0)
    comm = mccl.Communicator(1, mccl.get_unique_id(), 0, transport="cuda")
    assert comm.transport == "cuda" and comm.size == 1 and comm.device == 0
    x = torch.randn(100003, device="cuda")
    y = torch.empty_like(x)
    comm.all_reduce(x, y, op="avg")
    g = torch.empty_like(x)
    comm.all_gather(x, g)
    s = comm.empty(4096, torch.bfloat16)
    s.fill_(2.0)
    comm.all_reduce(s, op="sum")
    torch.cuda.synchronize()
    assert torch.equal(x, y) and torch.equal(x, g) and torch.all(s == 2.0)
    assert comm.peer_pointer(s, 0) == s.data_ptr()
    assert comm.launch_count >= 2 and comm.async_error() == 0
    assert "gpu" in comm.topo_xml()
    comm.finalize(); comm.destroy()


def test_graft_smoke():
    _require_cuda()
    import __graft_entry__ as entry
    entry.smoke()


@need2
def test_all_reduce_matrix_two_gpus():
    assert_all_ok(run_ranks(2, "matrix", worker="_gpu_worker.py", timeout=900))


@need2
def test_collectives_two_gpus():
    assert_all_ok(run_ranks(2, "collectives", worker="_gpu_worker.py", timeout=900))


@need2
def test_staging_with_small_stage_and_ipc_heap():
    # A 1 MB stage forces the chunked staging loops; IPC mode exercises the cudaMalloc + cudaIpc fallback.
    env = {"MCCL_STAGE_MB": "1", "MCCL_HEAP_MODE_IPC": "1"}
    assert_all_ok(run_ranks(2, "matrix", worker="_gpu_worker.py", env=env, args={"quick": True}, timeout=900))


@pytest.mark.skipif(NGPU < 4, reason="needs four GPUs")
def test_matrix_and_collectives_all_gpus():
    n = 8 if NGPU >= 8 else 4
    assert_all_ok(run_ranks(n, "matrix", worker="_gpu_worker.py", args={"quick": True}, timeout=1200))
    assert_all_ok(run_ranks(n, "collectives", worker="_gpu_worker.py", timeout=1200))


@pytest.mark.skipif(NGPU < 3, reason="needs three GPUs")
def test_odd_world_size():
    assert_all_ok(run_ranks(3, "matrix", worker="_gpu_worker.py", args={"quick": True}, timeout=900))


@need2
def test_split_and_ddp():
    assert_all_ok(run_ranks(min(NGPU, 4), "split_and_ddp", worker="_gpu_worker.py", timeout=600))


@need2
def test_device_wait_times_out_cleanly():
    # Bounded device waits, NVLS off, plain peer loads: a rank that sits out is reported, nothing hangs or traps.
    env = {"MCCL_DEVICE_TIMEOUT_MS": "1000", "MCCL_NVLS_ENABLE": "0"}
    assert_all_ok(run_ranks(2, "device_timeout", worker="_gpu_worker.py", env=env, timeout=120))


def test_sum_squares_and_clipped_step():
    _require_cuda()
    from mccl_b200.ops.optim import adamw_reference, fused_adamw_, scratch_floats, sum_squares_
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    out = torch.zeros(1, device=dev)
    for n in (1, 9, 65536, 65537, 3_000_001):
        x = torch.randn(n + 1, device=dev).to(torch.bfloat16)
        scratch = torch.zeros(scratch_floats(n), device=dev)
        for view in (x[:n], x[1:]):                        # the second view is not 16-byte aligned
            sum_squares_(view, out, scratch)
            ref = view.float().pow(2).sum()
            assert torch.allclose(out[0], ref, rtol=2e-5), (n, out.item(), ref.item())
            sum_squares_(view, out, scratch, accumulate=True)
            assert torch.allclose(out[0], 2 * ref, rtol=2e-5)
    # clipping inside the optimizer kernel equals scaling the gradient by min(1, max_norm/||g||)
    n = 4099
    master = torch.randn(n, device=dev); param = master.to(torch.bfloat16)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    rm, rma, rv = master.clone(), m.clone(), v.clone()
    grad = torch.randn(n, device=dev).to(torch.bfloat16)
    g2 = grad.clone()
    sum_squares_(grad, out, torch.zeros(scratch_floats(n), device=dev))
    fused_adamw_(param, master, m, v, grad, lr=1e-2, weight_decay=0.0, step=1, norm_sq=out, max_norm=1.0)
    scale = min(1.0, 1.0 / (g2.float().norm().item() + 1e-6))
    adamw_reference(rm, rma, rv, g2, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0, grad_scale=scale, step=1)
    torch.cuda.synchronize()
    assert torch.allclose(master, rm, rtol=1e-4, atol=1e-5)


def test_tcgen05_gemm_matches_fp32_reference():
    _require_cuda()
    from mccl_b200.ops import gemm as G
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    for (M, N, K) in [(128, 64, 64), (256, 448, 192), (1024, 3584, 1024), (384, 8192, 3584)]:
        x = (torch.randn(M, K, device=dev) * 0.5).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
        for epi in ("none", "silu"):
            y = G.gemm(x, w, epilogue=epi, two_sm=False)
            torch.cuda.synchronize()
            assert G.last_error() == 0
            ref = x.float() @ w.float().t()
            if epi == "silu":
                ref = torch.nn.functional.silu(ref)
            err = ((y.float() - ref).abs() / (ref.abs() + 1.0)).max().item()
            assert err < 1e-2, (M, N, K, epi, err)
    with pytest.raises(ValueError):
        G.gemm(torch.zeros(100, 64, device=dev, dtype=torch.bfloat16), torch.zeros(64, 64, device=dev, dtype=torch.bfloat16))


def test_two_sm_gemm_matches_fp32_reference():
    _require_cuda()
    from mccl_b200.ops import gemm as G
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    # the last two shapes leave a last wave of 4 and 8 tiles, which is cut along K over all SM pairs (split tail)
    for (M, N, K) in [(256, 64, 64), (256, 448, 192), (1024, 3584, 1024), (512, 8192, 3584), (8192, 256, 128),
                      (8192, 3584, 4096), (8192, 7168, 2048)]:
        x = (torch.randn(M, K, device=dev) * 0.5).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
        for epi in ("none", "silu", "none"):           # the repeat reuses the split tail's workspace: it must come back clean
            y = G.gemm(x, w, epilogue=epi, two_sm=True)
            torch.cuda.synchronize()
            assert G.last_error() == 0
            ref = x.float() @ w.float().t()
            if epi == "silu":
                ref = torch.nn.functional.silu(ref)
            err = ((y.float() - ref).abs() / (ref.abs() + 1.0)).max().item()
            assert err < 1e-2, (M, N, K, epi, err)


@need2
def test_fused_tp_ffn_one_sm_kernels():
    # the two-SM kernels are the default; MCCL_GEMM_2SM=0 selects the one-SM form
    assert_all_ok(run_ranks(2, "tp_ffn", worker="_gpu_worker.py", env={"MCCL_GEMM_2SM": "0"}, timeout=300))


@need2
def test_fused_tp_ffn_two_gpus():
    assert_all_ok(run_ranks(2, "tp_ffn", worker="_gpu_worker.py", timeout=300))
    assert_all_ok(run_ranks(2, "tp_ffn", worker="_gpu_worker.py", timeout=300,
                            args={"tokens": 2048, "hidden": 1024, "ffn": 7168}))


@pytest.mark.skipif(NGPU < 8, reason="needs eight GPUs")
def test_fused_tp_ffn_eight_gpus():
    assert_all_ok(run_ranks(8, "tp_ffn", worker="_gpu_worker.py", timeout=600,
                            args={"tokens": 8192, "hidden": 2048, "ffn": 8192}))


@need2
def test_calibration_and_trace(tmp_path):
    env = {"MCCL_CALIBRATE": "1", "MCCL_TRACE": str(tmp_path / "t")}
    assert_all_ok(run_ranks(2, "calibrate_and_trace", worker="_gpu_worker.py", env=env, timeout=300))


def test_probes_single_gpu():
    _require_cuda()
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for args in (["gpu"], ["kernels"], ["coll", "--op", "allreduce", "--transport", "cuda"]):
        r = subprocess.run([sys.executable, "-m", "mccl_b200.probe", *args], cwd=root, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, (args, r.stdout[-500:], r.stderr[-500:])


@need2
def test_large_messages():
    assert_all_ok(run_ranks(min(NGPU, 8) if NGPU in (2, 4, 8) else 2, "large_root_collectives", worker="_gpu_worker.py", timeout=600))


def test_fused_cross_entropy_matches_fp32_reference():
    _require_cuda()
    from mccl_b200.ops.loss import fused_cross_entropy
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    for rows, vocab, width in [(7, 1000, 1024), (64, 50257, 50304), (33, 129, 136)]:
        base = (torch.randn(rows, width, device=dev) * 3).to(torch.bfloat16)
        tgt = torch.randint(0, vocab, (rows,), device=dev)
        a = base.clone().requires_grad_(True)
        ref_in = base.float()[:, :vocab].clone().requires_grad_(True)
        ref = torch.nn.functional.cross_entropy(ref_in, tgt)
        (ref * 2.5).backward()
        # the kernel overwrites its input with the gradient, so feed it a copy that autograd tracks
        x = a * 1.0
        loss = fused_cross_entropy(x, tgt, vocab)
        (loss * 2.5).backward()
        torch.cuda.synchronize()
        assert abs(loss.item() - ref.item()) < 1e-4 * max(1.0, abs(ref.item())), (rows, vocab, loss.item(), ref.item())
        g = a.grad.float()
        assert torch.count_nonzero(g[:, vocab:]) == 0                       # padding columns get no gradient
        err = (g[:, :vocab] - ref_in.grad).abs().max().item()
        assert err < 1e-2 * ref_in.grad.abs().max().item() + 1e-6, (rows, vocab, err)


def test_fused_layer_norm_matches_fp32_reference():
    _require_cuda()
    from mccl_b200.ops.norm import FusedLayerNorm
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    for rows, d in [(5, 256), (777, 1024), (8192, 1024), (64, 512)]:
        ln = FusedLayerNorm(d).to(device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            ln.weight.copy_(torch.randn(d) * 0.5 + 1.0); ln.bias.copy_(torch.randn(d) * 0.1)
        x = (torch.randn(rows, d, device=dev) * 2 + 0.3).to(torch.bfloat16).requires_grad_(True)
        dy = torch.randn(rows, d, device=dev).to(torch.bfloat16)
        y = ln(x)
        y.backward(dy)
        xr = x.detach().float().requires_grad_(True)
        w, b = ln.weight.detach().float().requires_grad_(True), ln.bias.detach().float().requires_grad_(True)
        yr = torch.nn.functional.layer_norm(xr, (d,), w, b, ln.eps)
        yr.backward(dy.float())
        torch.cuda.synchronize()
        # outputs are rounded to bf16: compare relative to each value's magnitude
        assert ((y.float() - yr).abs() / (yr.abs() + 1.0)).max() < 1e-2
        assert ((x.grad.float() - xr.grad).abs() / (xr.grad.abs() + 1.0)).max() < 2e-2
        tol = 2e-2 * max(1.0, w.grad.abs().max().item())
        assert (ln.weight.grad.float() - w.grad).abs().max() < tol, (rows, d, (ln.weight.grad.float() - w.grad).abs().max().item())
        assert (ln.bias.grad.float() - b.grad).abs().max() < 2e-2 * max(1.0, b.grad.abs().max().item())
    # widths the kernel does not cover fall back to PyTorch
    ln = FusedLayerNorm(128).to(device=dev, dtype=torch.bfloat16)
    assert ln(torch.randn(4, 128, device=dev).to(torch.bfloat16)).shape == (4, 128)


@pytest.mark.parametrize("algo", ["twoshot", "oneshot", "ring", "tree"])
def test_emulated_ranks_all_reduce_on_one_gpu(algo):
    """The production kernel bodies with 2-8 emulated ranks in one cooperative launch on one GPU."""
    _require_cuda()
    from mccl_b200 import emu
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    for n in (2, 3, 8):
        for dtype in (torch.float32, torch.bfloat16, torch.int32):
            for numel in ((4096, 60000) if algo == "oneshot" else (4096, 1_000_003 if algo == "twoshot" else 1_000_000)):
                if algo in ("ring", "tree", "oneshot") and (numel * torch.empty((), dtype=dtype).element_size()) % 16:
                    continue
                for op in ("sum", "avg", "max"):
                    g = torch.Generator(device="cuda").manual_seed(n * 1000 + numel)
                    if dtype.is_floating_point:
                        xs = [(torch.rand(numel, generator=g, device=dev) * 2 - 1).to(dtype) for _ in range(n)]
                        st = torch.stack([x.double() for x in xs])
                    else:
                        xs = [torch.randint(-1000, 1000, (numel,), generator=g, device=dev, dtype=dtype) for _ in range(n)]
                        st = torch.stack([x.long() for x in xs])
                    ref = st.sum(0) if op in ("sum", "avg") else st.max(0).values
                    if op == "avg":
                        ref = ref / n if dtype.is_floating_point else torch.div(ref.to(dtype), n, rounding_mode="trunc")
                    emu.all_reduce(xs, op=op, algo=algo)
                    torch.cuda.synchronize()
                    for r, x in enumerate(xs):
                        if dtype.is_floating_point:
                            tol = {torch.float32: 1e-5, torch.bfloat16: 3e-2}[dtype] * (n if algo in ("ring", "tree") else 1)
                            err = ((x.double() - ref).abs() / (ref.abs() + 1.0)).max().item()
                            assert err <= tol, (algo, n, dtype, numel, op, r, err)
                        else:
                            assert torch.equal(x, ref.to(dtype)), (algo, n, dtype, numel, op, r)
                        assert torch.equal(x, xs[0]), "ranks must end with identical bytes"
    emu.destroy()


def test_emulated_one_shot_calls_of_mixed_sizes_stay_in_step():
    """Small and large one-shot calls run different grids; every CTA's call counter (which picks the half of the
    exchange slots a call uses) must advance all the same, or a later call could overwrite slots a peer still reads."""
    _require_cuda()
    from mccl_b200 import emu
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n = 4
    g = torch.Generator(device="cuda").manual_seed(11)
    for it, (kb, ctas) in enumerate([(32, 2), (128, 8), (64, 2), (72, 8), (64, 2), (16, 1), (128, 8), (32, 3)]):
        numel = kb * 1024 // 4
        xs = [torch.rand(numel, generator=g, device=dev) * 2 - 1 for _ in range(n)]
        ref = torch.stack([x.double() for x in xs]).sum(0)
        emu.all_reduce(xs, op="sum", algo="oneshot", ctas=ctas)
        torch.cuda.synchronize()
        for x in xs:
            assert ((x.double() - ref).abs() / (ref.abs() + 1.0)).max().item() <= 1e-5, (it, kb, ctas)
            assert torch.equal(x, xs[0])
        for r in range(n):
            assert emu.one_shot_counters(r) == [it + 1] * 8, (it, r, emu.one_shot_counters(r))
    emu.destroy()


def test_emulated_ranks_misaligned_buffers():
    """Buffers that do not start on a 16-byte boundary take the element-granular path of the two-shot kernel."""
    _require_cuda()
    from mccl_b200 import emu
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    for dtype, numel in ((torch.float32, 100_003), (torch.bfloat16, 77_777), (torch.int32, 5)):
        n = 4
        g = torch.Generator(device="cuda").manual_seed(7)
        bases = [torch.zeros(numel + 3, device=dev, dtype=dtype) for _ in range(n)]
        views = [b[1:numel + 1] for b in bases]                       # 2 or 4 bytes past a 16-byte boundary
        for v in views:
            v.copy_((torch.rand(numel, generator=g, device=dev) * 200 - 100).to(dtype))
        ref = torch.stack([v.double() for v in views]).sum(0)
        emu.all_reduce(views, op="sum", algo="twoshot")
        torch.cuda.synchronize()
        for b, v in zip(bases, views):
            err = ((v.double() - ref).abs() / (ref.abs() + 1.0)).max().item()
            assert err <= (3e-2 if dtype == torch.bfloat16 else 1e-5), (dtype, err)
            assert b[0] == 0 and b[numel + 1] == 0 and b[numel + 2] == 0     # neighbours untouched
    emu.destroy()


def test_emulated_ring_and_tree_phases():
    """The partial forms the cuda transport uses for ring all-gather / reduce-scatter and tree broadcast / reduce."""
    _require_cuda()
    from mccl_b200 import emu
    import ctypes as C
    lib = __import__("mccl_b200").load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    for n in (2, 3, 8):
        part = 4096 + 8 * n                                         # elements per part, a multiple of 4 (16 bytes of fp32)
        g = torch.Generator(device="cuda").manual_seed(n)
        # ring gather steps, shift 1: rank r starts with part r filled, everyone ends with all parts
        truth = torch.rand(n * part, generator=g, device=dev)
        bufs = [torch.full((n * part,), -1.0, device=dev) for _ in range(n)]
        for r in range(n):
            bufs[r][r * part:(r + 1) * part] = truth[r * part:(r + 1) * part]
        emu.phases(bufs, "ring", 2, shift=1)
        torch.cuda.synchronize()
        assert all(torch.equal(b, truth) for b in bufs), ("ring gather", n)
        # ring reduce steps, shift 1: rank r ends owning the fully reduced part r
        ins = [torch.rand(n * part, generator=g, device=dev) for _ in range(n)]
        ref = torch.stack([x.double() for x in ins]).sum(0)
        work = [x.clone() for x in ins]
        emu.phases(work, "ring", 1, shift=1, op="avg")
        torch.cuda.synchronize()
        for r in range(n):
            got = work[r][r * part:(r + 1) * part].double()
            assert ((got - ref[r * part:(r + 1) * part] / n).abs() / (ref[r * part:(r + 1) * part].abs() / n + 1)).max() < 1e-5, ("ring reduce", n, r)
        # tree up: each half ends reduced at its tree's root; tree down: the roots' halves reach everyone
        roots = []
        for t in (0, 1):
            for r in range(n):
                out = (C.c_int * 6)()
                lib.mcclDbgDtree(n, r, out)
                if out[3 * t] < 0:
                    roots.append(r)
        half = (n * part // 4 // 2) * 4
        work = [x.clone() for x in ins]
        emu.phases(work, "tree", 1)
        torch.cuda.synchronize()
        assert ((work[roots[0]][:half].double() - ref[:half]).abs() / (ref[:half].abs() + 1)).max() < 1e-5, ("tree up A", n)
        assert ((work[roots[1]][half:].double() - ref[half:]).abs() / (ref[half:].abs() + 1)).max() < 1e-5, ("tree up B", n)
        bufs = [torch.full((n * part,), -1.0, device=dev) for _ in range(n)]
        bufs[roots[0]][:half] = truth[:half]
        bufs[roots[1]][half:] = truth[half:]
        emu.phases(bufs, "tree", 2)
        torch.cuda.synchronize()
        assert all(torch.equal(b, truth) for b in bufs), ("tree down", n)
    emu.destroy()


@need2
def test_forced_ring_and_tree_for_other_collectives():
    assert_all_ok(run_ranks(min(NGPU, 4), "forced_ring_tree", worker="_gpu_worker.py", timeout=600))


@need2
def test_torch_distributed_backend_on_gpus(tmp_path):
    assert_all_ok(run_ranks(2, "c10d_backend_gpu", worker="_gpu_worker.py", args={"rendezvous": str(tmp_path / "rdv")}, timeout=300))


@need2
def test_gather_scatter_alltoallv_on_gpus():
    assert_all_ok(run_ranks(min(NGPU, 4), "rooted_and_ragged_gpu", worker="_gpu_worker.py", timeout=300))


@need2
def test_trainable_fused_tensor_parallel_mlp():
    assert_all_ok(run_ranks(2, "tp_mlp_trainable", worker="_gpu_worker.py", timeout=600))


@need2
def test_fused_moe_dispatch_and_combine():
    assert_all_ok(run_ranks(min(NGPU, 4), "moe_fused", worker="_gpu_worker.py", timeout=600))


@need2
def test_model_parallel_layers_on_gpus():
    assert_all_ok(run_ranks(2, "parallel_layers_gpu", worker="_gpu_worker.py", timeout=600))


@need2
def test_ddp_sharded_optimizer_on_gpus():
    assert_all_ok(run_ranks(min(NGPU, 4), "ddp_sharded", worker="_gpu_worker.py", timeout=600))


@need2
def test_collectives_replay_from_a_cuda_graph():
    assert_all_ok(run_ranks(2, "graph_capture", worker="_gpu_worker.py", timeout=300))


@need2
def test_composed_ring_and_tree_forms():
    assert_all_ok(run_ranks(min(NGPU, 4), "forced_ring_tree", worker="_gpu_worker.py", args={"composed": True}, timeout=900))


@need2
def test_rooted_collectives_spread_over_all_ranks():
    assert_all_ok(run_ranks(min(NGPU, 4), "rooted_spread", worker="_gpu_worker.py", env={"MCCL_NVLS_SPREAD": "1"}, timeout=600))


@need2
def test_ddp_step_recorded_in_a_cuda_graph():
    assert_all_ok(run_ranks(2, "ddp_graphed", worker="_gpu_worker.py", timeout=600))


def test_graphed_step_on_one_gpu_matches_eager():
    _require_cuda()
    from mccl_b200.models.gpt2 import GPT2, GPT2Config
    from mccl_b200.parallel.ddp import DistributedDataParallel
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = GPT2Config.tiny()
    batches = torch.randint(0, cfg.vocab_size, (3, 4, cfg.seq_len + 1), generator=torch.Generator().manual_seed(3)).to(dev)

    def build():
        torch.manual_seed(0)
        return DistributedDataParallel(GPT2(cfg).to(device=dev, dtype=torch.bfloat16), None)

    eager, ref = build(), []
    for i in range(6):
        t = batches[i % 3]
        loss = eager(t[:, :-1], t[:, 1:]); loss.backward(); eager.step(lr=3e-3, max_grad_norm=1.0)
        ref.append(loss.item())
    ddp = build()
    step = ddp.graphed_step((batches[0][:, :-1], batches[0][:, 1:]), lr=3e-3, max_grad_norm=1.0, warmup=1)
    got = [ref[0]] + [step(batches[i % 3][:, :-1], batches[i % 3][:, 1:]).item() for i in range(1, 6)]
    for a, b in zip(ref, got):
        assert abs(a - b) < 2e-2 * max(1.0, abs(a)), (ref, got)
    assert got[-1] < got[1] and ddp.step_count == 6


@need2
def test_symmetric_buffer_contract_is_checked_on_request():
    assert_all_ok(run_ranks(2, "symmetry_check", worker="_gpu_worker.py", env={"MCCL_CHECK_SYMMETRY": "1"}, timeout=300))


@need2
def test_group_of_all_reduce_calls_is_one_launch():
    assert_all_ok(run_ranks(min(NGPU, 4), "grouped_allreduce", worker="_gpu_worker.py", timeout=300))


@need2
def test_register_user_buffer():
    assert_all_ok(run_ranks(2, "register_user_buffer", worker="_gpu_worker.py", timeout=300))
