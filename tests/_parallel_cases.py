"""Model-parallel layer and pipeline cases shared by the cpu (tcp transport) and gpu (cuda transport) workers."""


def layers_case(comm, RANK, WORLD, dev, atol=2e-5):
    """Tensor / sequence / expert parallel layers on the tcp transport against single-process restatements:
    outputs and every gradient (inputs and weight shards)."""
    import torch
    import torch.nn.functional as F
    from mccl_b200.parallel import layers as PL
    n, r = WORLD, RANK
    close = lambda a, b, what: (torch.allclose(a, b, atol=atol, rtol=50 * atol) or (_ for _ in ()).throw(AssertionError((what, (a - b).abs().max().item()))))
    gen = torch.Generator().manual_seed(3)
    T, hid, ffn = 6 * n, 16, 8 * n
    x_full = torch.randn(T, hid, generator=gen).to(dev)
    wu, wd = (torch.randn(ffn, hid, generator=gen) * 0.3).to(dev), (torch.randn(hid, ffn, generator=gen) * 0.3).to(dev)
    bu, bd = (torch.randn(ffn, generator=gen) * 0.1).to(dev), (torch.randn(hid, generator=gen) * 0.1).to(dev)
    tgt = torch.randn(T, hid, generator=gen).to(dev)
    # single process
    xf = x_full.clone().requires_grad_(True)
    wuf, wdf, buf, bdf = (t.clone().requires_grad_(True) for t in (wu, wd, bu, bd))
    yf = F.linear(F.silu(F.linear(xf, wuf, buf)), wdf, bdf)
    (yf * tgt).sum().backward()
    blk, m = T // n, ffn // n
    for sp in (True, False):
        mlp = PL.TensorParallelMLP(comm, hid, ffn, bias=True, sequence_parallel=sp, device=dev)
        mlp.up.load_full(wu, bu); mlp.down.load_full(wd, bd)
        x = (x_full[r * blk:(r + 1) * blk] if sp else x_full).clone().requires_grad_(True)
        y = mlp(x)
        t_loc = tgt[r * blk:(r + 1) * blk] if sp else tgt
        (y * t_loc).sum().backward()
        close(y, yf[r * blk:(r + 1) * blk] if sp else yf, ("mlp out", sp))
        close(x.grad, xf.grad[r * blk:(r + 1) * blk] if sp else xf.grad, ("mlp dx", sp))
        close(mlp.up.weight.grad, wuf.grad[r * m:(r + 1) * m], ("mlp dWup", sp))
        close(mlp.up.bias.grad, buf.grad[r * m:(r + 1) * m], ("mlp dbup", sp))
        close(mlp.down.weight.grad, wdf.grad[:, r * m:(r + 1) * m], ("mlp dWdown", sp))
        if not sp:
            close(mlp.down.bias.grad, bdf.grad, ("mlp dbdown", sp))
        else:                                   # a share per rank: summed over ranks it is the full gradient
            g = mlp.down.bias.grad.clone(); comm.all_reduce(g, op="sum")
            close(g, bdf.grad, ("mlp dbdown summed", sp))

    # Ulysses attention
    S, H, D = 4 * n, 2 * n, 8
    q, k, v, tg = (torch.randn(S, H, D, generator=gen).to(dev) for _ in range(4))
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    of = PL.attention_reference(qf, kf, vf, causal=True)
    (of * tg).sum().backward()
    sb = S // n
    ql, kl, vl = (t[r * sb:(r + 1) * sb].clone().requires_grad_(True) for t in (q, k, v))
    o = PL.UlyssesAttention(comm, H, causal=True)(ql, kl, vl)
    (o * tg[r * sb:(r + 1) * sb]).sum().backward()
    close(o, of[r * sb:(r + 1) * sb], "ulysses out")
    for name, a, b in (("dq", ql, qf), ("dk", kl, kf), ("dv", vl, vf)):
        close(a.grad, b.grad[r * sb:(r + 1) * sb], "ulysses " + name)

    # ring (context parallel) attention on the same tensors, with and without the causal mask, odd head count allowed
    for causal in (True, False):
        q3, k3, v3 = (t[:, :3].contiguous() for t in (q, k, v))
        qf, kf, vf = (t.clone().requires_grad_(True) for t in (q3, k3, v3))
        of = PL.attention_reference(qf, kf, vf, causal=causal)
        (of * tg[:, :3]).sum().backward()
        ql, kl, vl = (t[r * sb:(r + 1) * sb].clone().requires_grad_(True) for t in (q3, k3, v3))
        o = PL.RingAttention(comm, causal=causal)(ql, kl, vl)
        (o * tg[r * sb:(r + 1) * sb, :3]).sum().backward()
        close(o, of[r * sb:(r + 1) * sb], ("ring out", causal))
        for name, a, b in (("dq", ql, qf), ("dk", kl, kf), ("dv", vl, vf)):
            close(a.grad, b.grad[r * sb:(r + 1) * sb], ("ring " + name, causal))

    # expert parallel mixture of experts
    e_loc, cap = 2, 2
    E = e_loc * n
    Tm = E * cap + 3                              # more tokens than slots: some are dropped
    router_w = torch.randn(E, hid, generator=gen).to(dev)
    w_in_all, w_out_all = (torch.randn(E, ffn, hid, generator=gen) * 0.3).to(dev), (torch.randn(E, hid, ffn, generator=gen) * 0.3).to(dev)
    xs = [torch.randn(Tm, hid, generator=gen).to(dev) for _ in range(n)]
    moe = PL.ExpertParallelMoE(comm, hid, ffn, e_loc, cap, device=dev)
    with torch.no_grad():
        moe.router.weight.copy_(router_w)
        moe.w_in.copy_(w_in_all[r * e_loc:(r + 1) * e_loc]); moe.w_out.copy_(w_out_all[r * e_loc:(r + 1) * e_loc])
    xm = xs[r].clone().requires_grad_(True)
    ym = moe(xm)
    ym.sum().backward()
    rw, wi, wo = (t.clone().requires_grad_(True) for t in (router_w, w_in_all, w_out_all))
    xr = [t.clone().requires_grad_(True) for t in xs]
    refs = [PL.moe_reference(xr[i], rw, wi, wo, cap) for i in range(n)]
    sum(t.sum() for t in refs).backward()
    close(ym, refs[r].detach(), "moe out")
    assert (ym.abs().sum(-1) == 0).any(), "the capacity rule dropped nothing"
    close(xm.grad, xr[r].grad, "moe dx")
    close(moe.w_in.grad, wi.grad[r * e_loc:(r + 1) * e_loc], "moe dW_in")
    close(moe.w_out.grad, wo.grad[r * e_loc:(r + 1) * e_loc], "moe dW_out")
    g = moe.router.weight.grad.clone(); comm.all_reduce(g, op="sum")       # the router is replicated: sum the shares
    close(g, rw.grad, "moe d router")



def pipeline_case(comm, RANK, WORLD, dev, atol=2e-5):
    """One stage per rank, 1F1B over Send / Recv: loss and parameter gradients equal single-process training on
    the whole batch, for fewer, as many and more micro-batches than stages."""
    import torch
    import torch.nn as nn
    from mccl_b200.parallel.pipeline import PipelineStage
    torch.manual_seed(0)
    width, micro = 12, 3
    full = nn.ModuleList([nn.Sequential(nn.Linear(width, width), nn.Tanh()) for _ in range(WORLD)]).to(dev)
    mine = full[RANK]
    stage = PipelineStage(comm, mine, (micro, width))
    loss_fn = lambda y, t: ((y - t) ** 2).mean()
    gen = torch.Generator().manual_seed(9)
    for n_micro in (1, WORLD, 2 * WORLD + 1):
        xs = [torch.randn(micro, width, generator=gen).to(dev) for _ in range(n_micro)]
        ts = [torch.randn(micro, width, generator=gen).to(dev) for _ in range(n_micro)]
        for p in full.parameters():
            p.grad = None
        loss = stage.run(xs if RANK == 0 else None, ts if RANK == WORLD - 1 else None, loss_fn, n_micro)
        got = [p.grad.clone() for p in mine.parameters()]
        for p in full.parameters():
            p.grad = None
        ref = 0.0
        for x, t in zip(xs, ts):
            y = x
            for m in full:
                y = m(y)
            l = loss_fn(y, t) / n_micro
            l.backward()
            ref += l.item()
        if RANK == WORLD - 1:
            assert abs(loss.item() - ref) < 10 * atol, (n_micro, loss.item(), ref)
        for g, p in zip(got, mine.parameters()):
            assert torch.allclose(g, p.grad, atol=atol, rtol=50 * atol), (n_micro, (g - p.grad).abs().max().item())


def llama_case(comm, RANK, WORLD, dev, atol=2e-5):
    """The tensor-parallel Llama-style decoder (replicated and sequence-parallel residual stream) against the same
    model on a communicator of size 1: loss and every gradient."""
    import torch
    import mccl_b200 as mccl
    from mccl_b200.models.llama import Llama, LlamaConfig
    cfg = LlamaConfig.tiny()
    cfg.d_ff = 32 * WORLD
    cfg.n_head = 2 * WORLD
    cfg.d_model = 16 * cfg.n_head
    one = mccl.Communicator(1, mccl.get_unique_id(), 0, transport=comm.transport)
    torch.manual_seed(0)
    ref = Llama(cfg, one).to(dev)
    state = {k: v.detach().clone() for k, v in ref.named_parameters()}
    g = torch.Generator().manual_seed(4)
    tokens = torch.randint(0, cfg.vocab_size, (2 * WORLD, cfg.seq_len + 1), generator=g).to(dev)
    idx, tgt = tokens[:, :-1], tokens[:, 1:]
    lref = ref(idx, tgt)
    lref.backward()
    n, r = WORLD, RANK
    for sp in (False, True):
        model = Llama(cfg, comm, sequence_parallel=sp).to(dev)
        model.load_full(state)
        loss = model(idx, tgt)
        loss.backward()
        model.reduce_replicated_grads()
        assert abs(loss.item() - lref.item()) < 10 * atol, (sp, loss.item(), lref.item())
        full = dict(ref.named_parameters())
        for name, p in model.named_parameters():
            want = full[name].grad
            leaf = name.split(".")[-2]
            if leaf in ("q", "k", "v", "gate", "up"):
                m = want.shape[0] // n
                want = want[r * m:(r + 1) * m]
            elif leaf in ("o", "down"):
                m = want.shape[1] // n
                want = want[:, r * m:(r + 1) * m]
            assert torch.allclose(p.grad, want, atol=atol, rtol=50 * atol), (sp, name, (p.grad - want).abs().max().item())
    one.destroy()


def fsdp_case(comm, RANK, WORLD, dev, atol=2e-5):
    """Fully sharded blocks (parameters gathered just in time, gradients reduce-scattered, optimizer on the shards)
    follow single-process training on the concatenated batch; the state per rank is 1/world."""
    import torch
    import torch.nn as nn
    from mccl_b200.parallel.fsdp import FullyShardedStack
    def make():
        torch.manual_seed(0)
        return [m.to(dev) for m in [nn.Sequential(nn.Linear(24, 40), nn.Tanh(), nn.Linear(40, 24)) for _ in range(3)] + [nn.Sequential(nn.Linear(24, 7))]]
    fsdp = FullyShardedStack(make(), comm)
    ref = nn.Sequential(*make())
    assert sum(p.numel() for p in fsdp.shard_parameters()) * WORLD <= sum(p.numel() for p in ref.parameters()) + 4 * 8 * WORLD * 8
    o1, o2 = torch.optim.Adam(fsdp.shard_parameters(), lr=1e-2), torch.optim.Adam(ref.parameters(), lr=1e-2)
    g = torch.Generator().manual_seed(8)
    for step in range(4):
        x, y = torch.randn(3 * WORLD, 24, generator=g).to(dev), torch.randn(3 * WORLD, 7, generator=g).to(dev)
        o1.zero_grad(); o2.zero_grad()
        torch.nn.functional.mse_loss(fsdp(x[3 * RANK:3 * RANK + 3]), y[3 * RANK:3 * RANK + 3]).backward()
        torch.nn.functional.mse_loss(ref(x), y).backward()
        o1.step(); o2.step()
    for flat, block in zip(fsdp.full_state(), ref):
        want = torch.cat([torch.nn.functional.pad(p.detach().reshape(-1), (0, (-p.numel()) % 8)) for p in block.parameters()])
        got = flat[: want.numel()]
        assert torch.allclose(got, want, atol=atol, rtol=50 * atol), (got - want).abs().max().item()
