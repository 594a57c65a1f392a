"""Fused peer-memory expert parallelism on real GPUs.  Every multi-rank run computes the layer
six ways and compares them: one-hop and two-hop under the overlap schedule and under the
remote-read schedule (all four bit for bit), the ``torch.distributed`` arm, and a dense fp32
PyTorch oracle of the same layer (forward, input, gate and weight gradients, within tolerance)."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, queue, M, rpn=1):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        _body(rank, world, queue, M, rpn)
        dist.barrier()
    except Exception as exc:  # noqa: BLE001  (the parent must hear of it instead of waiting)
        import traceback
        queue.put((rank, "error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))
    finally:
        dist.destroy_process_group()


CAPACITY = 1400          # rows per rank the arena is sized for; every rank's T stays below it


def _fp32_oracle(rank, world, x0, idx, gates0, gy, w13_all, w2_all, dev, keep=None):
    """The layer as plain fp32 PyTorch over ALL ranks' tokens and ALL experts:
    ``y[t] = sum_j gate[t, j] * (silu(x W13a) * (x W13b)) W2`` of expert ``idx[t, j]``; autograd gives
    every gradient.  Returns this rank's slices, in the order of the fused results."""
    import torch.distributed as dist
    import torch.nn.functional as F
    parts = [None] * world
    mask = torch.ones_like(gates0) if keep is None else keep.to(gates0.dtype)
    dist.all_gather_object(parts, (x0.cpu(), idx.cpu(), gates0.cpu(), gy.cpu(), mask.cpu()))
    lo = sum(p[0].shape[0] for p in parts[:rank])
    hi = lo + parts[rank][0].shape[0]
    x = torch.cat([p[0] for p in parts]).float().to(dev).requires_grad_(True)
    ids = torch.cat([p[1] for p in parts]).to(dev)
    gates = torch.cat([p[2] for p in parts]).float().to(dev).requires_grad_(True)
    g_out = torch.cat([p[3] for p in parts]).float().to(dev)
    kept = torch.cat([p[4] for p in parts]).float().to(dev)      # 0 for picks beyond capacity
    w13 = w13_all.float().to(dev).requires_grad_(True)
    w2 = w2_all.float().to(dev).requires_grad_(True)
    y = torch.zeros_like(x)
    for e in range(w13.shape[0]):
        tok, col = (ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        a, b = (x[tok] @ w13[e]).chunk(2, dim=-1)
        y = y.index_add(0, tok, (gates[tok, col] * kept[tok, col]).unsqueeze(1)
                        * ((F.silu(a) * b) @ w2[e]))
    y.backward(g_out)
    epr = w13.shape[0] // world
    own = slice(rank * epr, (rank + 1) * epr)
    return [t.detach().float().cpu() for t in
            (y[lo:hi], x.grad[lo:hi], gates.grad[lo:hi], w13.grad[own], w2.grad[own])]


def _body(rank, world, queue, M, rpn):
    from terracemoe_simulator_b200 import ops
    from terracemoe_simulator_b200.parallel import fused as fz
    from terracemoe_simulator_b200.parallel.ep import ep_moe_forward
    from terracemoe_simulator_b200.routing import TRouteConfig, t_route
    assert ops.custom_ops_enabled()
    dev = torch.device("cuda", rank)
    E, k, H, d, T = 16, 4, 256, 128, 1000 + 37 * rank
    n_groups = max(world // rpn, 2)
    cfg = TRouteConfig(E, n_groups, k, M)
    g = torch.Generator().manual_seed(0)
    w13_all = (torch.randn(E, H, 2 * d, generator=g) * H ** -0.5).bfloat16()
    w2_all = (torch.randn(E, d, H, generator=g) * d ** -0.5).bfloat16()
    epr = E // world
    gx = torch.Generator().manual_seed(10 + rank)
    x0 = torch.randn(T, H, generator=gx).bfloat16().to(dev)
    aff = torch.rand(T, E, generator=gx).to(dev)
    gy = torch.randn(T, H, generator=gx).bfloat16().to(dev)
    idx, gates0, _ = t_route(aff, torch.zeros(E, device=dev), cfg)
    assert 1000 + 37 * (world - 1) <= CAPACITY
    # the context the environment asks for (default: the overlap schedule; a token pipeline when
    # TERRACE_EP_PIPELINE is set) and the remote-read schedule as the second arm
    fctx = fz.make_context(cfg, H, d, CAPACITY, world=world, rank=rank, rpn=rpn, device=dev)
    pull = fz.FusedEPContext(cfg, H, d, CAPACITY, world=world, rank=rank, rpn=rpn, device=dev,
                             overlap=False)
    res = {}
    hops = ["one_hop", "two_hop"] if world > 1 else ["one_hop"]
    arms = [(m, fctx, m) for m in hops] + [("pull_" + m, pull, m) for m in hops]
    for name, ctx, mode in arms + [("ref", None, None)]:
        x = x0.clone().requires_grad_(True)
        gates = gates0.clone().requires_grad_(True)
        a = w13_all[rank * epr:(rank + 1) * epr].to(dev).requires_grad_(True)
        b = w2_all[rank * epr:(rank + 1) * epr].to(dev).requires_grad_(True)
        for _ in range(2):              # twice: arena, flags and streams are reused
            for t in (x, gates, a, b):
                t.grad = None
            if name == "ref":
                if world == 1:
                    y = ops.moe_experts_local(x, idx, gates, a, b, cfg.group_size)
                else:
                    y = ep_moe_forward(x, idx, gates, a, b, world, E, rpn=rpn)
            else:
                y = fz.run_fused(ctx, x, idx, gates, a, b, mode=mode)
            y.backward(gy)
        torch.cuda.synchronize()
        res[name] = [t.detach().float().cpu() for t in (y, x.grad, gates.grad, a.grad, b.grad)]
    res["oracle"] = _fp32_oracle(rank, world, x0, idx, gates0, gy, w13_all, w2_all, dev)
    echo = fz.fused_dispatch_combine(fctx, x0, idx, gates0, mode=hops[-1])
    torch.cuda.synchronize()
    status = fctx.take_status() or ops.take_status(rank)
    bad = fctx.check_canaries() or pull.check_canaries()
    if not status and bad:            # a store went past the end of an arena section
        status = 7700 + (bad[0] if isinstance(bad[0], int) else bad[0][1])
    queue.put((rank, res, echo.float().cpu(), x0.float().cpu(), status,
               dict(fz.LIVE)))


def _run(world, M, port, rpn=1):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, M, rpn)) for r in range(world)]
    for p in procs:
        p.start()
    out, failed = [], None
    try:
        for _ in range(world):
            item = q.get(timeout=300)
            if item[1] == "error":
                failed = item
                break
            out.append(item)
    finally:
        for p in procs:
            p.join(timeout=30 if failed is None else 10)
        for p in procs:
            if p.is_alive():
                p.terminate()
    if failed is not None:
        raise AssertionError(f"rank {failed[0]} failed: {failed[2]}")
    return sorted(out, key=lambda t: t[0])


def _close(a, b, tol=5e-2):
    scale = b.abs().max().item() + 1e-6
    torch.testing.assert_close(a, b, rtol=tol, atol=tol * scale)


def _check_ranks(out, world, *, pipeline: int = 1):
    """Every rank: status 0; all fused arms bit-identical (weight gradients within rounding when
    token slices sum partial results); fused against the NCCL arm and the fp32 oracle."""
    hops = ["one_hop", "two_hop"] if world > 1 else ["one_hop"]
    for rank, res, echo, x0, status, live in out:
        assert status == 0, (rank, status)
        for m in hops:
            assert live[m + "_fwd"] >= 2 and live[m + "_bwd"] >= 2
        if pipeline == 1:
            assert live["overlap_fwd"] >= 2 * len(hops) and live["overlap_bwd"] >= 2 * len(hops)
            assert live["chunk_pushes"] > 0
        base = res["one_hop"]
        for name in ["two_hop"] * (world > 1):
            for a, b in zip(base, res[name]):
                assert torch.equal(a, b), "one-hop and two-hop fused paths must agree bit for bit"
        for name in ["pull_" + m for m in hops]:
            for i, (a, b) in enumerate(zip(base, res[name])):
                if pipeline > 1 and i >= 2:      # sums of per-slice partial results
                    _close(a, b, 2e-2)
                elif i == 2 and world == 1:
                    _close(a, b, 1e-2)
                else:
                    assert torch.equal(a, b), f"schedules disagree on tensor {i} ({name})"
        for i, (a, b) in enumerate(zip(base, res["ref"])):
            if world == 1 and i != 2:
                assert torch.equal(a, b)
            else:
                _close(a, b, 1e-2 if world == 1 else 5e-2)
        for a, b in zip(base, res["oracle"]):
            _close(a, b)
        # echo: every token gets sum_j gate_j * x = x (gates sum to one) up to bf16 rounding
        _close(echo, x0, 2e-2)


def test_fused_world1_equals_local_kernels(native_ops):
    _check_ranks(_run(1, 1, 29701), 1)


@pytest.mark.parametrize("M", [2, 1])
def test_fused_world2_one_hop_two_hop(native_ops, M):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _check_ranks(_run(2, M, 29703 + M), 2)


@pytest.mark.parametrize("world,rpn,M", [(4, 2, 2), (8, 2, 2), (8, 4, 2)])
def test_fused_groups_of_several_gpus(native_ops, world, rpn, M):
    """Logical groups of R > 1 GPUs: Hop B really crosses GPUs inside the group."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _check_ranks(_run(world, M, 29720 + world + rpn, rpn=rpn), world)


def _capacity_worker(rank, world, port, queue, rpn):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        from terracemoe_simulator_b200 import ops
        from terracemoe_simulator_b200.layer import apply_capacity
        from terracemoe_simulator_b200.parallel import fused as fz
        from terracemoe_simulator_b200.routing import TRouteConfig, expert_load, t_route
        dev = torch.device("cuda", rank)
        E, k, H, d, T, factor = 16, 4, 256, 128, 900, 0.7
        cfg = TRouteConfig(E, max(world // rpn, 2), k, 2)
        g = torch.Generator().manual_seed(0)
        w13_all = (torch.randn(E, H, 2 * d, generator=g) * H ** -0.5).bfloat16()
        w2_all = (torch.randn(E, d, H, generator=g) * d ** -0.5).bfloat16()
        epr = E // world
        gx = torch.Generator().manual_seed(20 + rank)
        x0 = torch.randn(T, H, generator=gx).bfloat16().to(dev)
        # skewed affinities, so that some experts overflow their capacity
        aff = (torch.rand(T, E, generator=gx) * torch.linspace(0.4, 1.0, E)).to(dev)
        gy = torch.randn(T, H, generator=gx).bfloat16().to(dev)
        idx, gates0, _ = t_route(aff, torch.zeros(E, device=dev), cfg)
        loads = [torch.zeros(E, device=dev) for _ in range(world)]
        dist.all_gather(loads, expert_load(idx, E))
        prior = sum(loads[:rank], torch.zeros(E, device=dev)).long()
        _, keep, cap = apply_capacity(idx, gates0, E, factor, n_tokens_global=T * world,
                                      prior_counts=prior)
        res = {}
        for name, overlap in (("overlap", True), ("pull", False)):
            ctx = fz.FusedEPContext(cfg, H, d, T, world=world, rank=rank, rpn=rpn, device=dev,
                                    overlap=overlap)
            for mode in ("one_hop", "two_hop"):
                x = x0.clone().requires_grad_(True)
                gates = gates0.clone().requires_grad_(True)
                a = w13_all[rank * epr:(rank + 1) * epr].to(dev).requires_grad_(True)
                b = w2_all[rank * epr:(rank + 1) * epr].to(dev).requires_grad_(True)
                y = fz.run_fused(ctx, x, idx, gates, a, b, mode=mode, capacity_factor=factor)
                y.backward(gy)
                torch.cuda.synchronize()
                res[f"{name}_{mode}"] = [t.detach().float().cpu()
                                         for t in (y, x.grad, gates.grad, a.grad, b.grad)]
        res["oracle"] = _fp32_oracle(rank, world, x0, idx, gates0, gy, w13_all, w2_all, dev,
                                     keep=keep)
        status = ops.take_status(rank)
        queue.put((rank, res, keep.cpu(), int((~keep).sum()), status, cap))
        dist.barrier()
    except Exception as exc:  # noqa: BLE001
        import traceback
        queue.put((rank, "error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,rpn", [(2, 1), (4, 2)])
def test_fused_capacity_on_the_device_matches_apply_capacity(native_ops, world, rpn):
    """Capacity factor inside the plan kernel: the dropped picks are exactly those the layer-level
    oracle drops (zero gate gradient there, non-zero elsewhere), the four fused arms agree bit
    for bit, and outputs and gradients match the fp32 oracle with the oracle's gates zeroed."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_capacity_worker, args=(r, world, 29850 + world, q, rpn))
             for r in range(world)]
    for p in procs:
        p.start()
    out = []
    try:
        for _ in range(world):
            out.append(q.get(timeout=300))
    finally:
        for p in procs:
            p.join(timeout=30)
        for p in procs:
            if p.is_alive():
                p.terminate()
    total_dropped = 0
    for item in out:
        assert item[1] != "error", item[2]
        rank, res, keep, dropped, status, cap = item
        assert status == 0, (rank, status)          # a dropped pick is not an error
        total_dropped += dropped
        base = res["overlap_one_hop"]
        for name in ("overlap_two_hop", "pull_one_hop", "pull_two_hop"):
            for a, b in zip(base, res[name]):
                assert torch.equal(a, b), name
        for a, b in zip(base, res["oracle"]):
            _close(a, b)
        # the gate gradient is exactly zero where, and only where, the oracle drops the pick
        assert bool((base[2][~keep] == 0).all())
        assert float((base[2][keep] != 0).float().mean()) > 0.99
    assert total_dropped > 0


@pytest.mark.parametrize("chunks", ["1", "4"])
def test_fused_world2_other_chunk_counts(native_ops, monkeypatch, chunks):
    """One push launch (no overlap window) and four: same bits as two."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    monkeypatch.setenv("TERRACE_EP_CHUNKS", chunks)
    _check_ranks(_run(2, 2, 29740 + int(chunks)), 2)


def _model_worker(rank, world, port, queue):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        from terracemoe_simulator_b200.parallel import fused as fz
        from terracemoe_simulator_b200.parallel import fused_model as fm
        from terracemoe_simulator_b200.routing import TRouteConfig, t_route
        dev = torch.device("cuda", rank)
        E, k, H, T = 16, 4, 256, 300 + 11 * rank
        cfg = TRouteConfig(E, max(world, 2), k, 2)
        g = torch.Generator().manual_seed(40 + rank)
        x = torch.randn(T, H, generator=g).bfloat16().to(dev)
        idx, gates, _ = t_route(torch.rand(T, E, generator=g).to(dev), torch.zeros(E, device=dev), cfg)
        fctx = fz.FusedEPContext(cfg, H, 128, 400, world=world, rank=rank, rpn=1, device=dev)
        ep = fctx.next_epoch()
        p = fz._plan(fctx, idx, gates, "one_hop", ep)
        fz._dispatch(fctx, p, x, "one_hop", ep)
        torch.cuda.synchronize()
        gathered = [None] * world
        dist.all_gather_object(gathered, idx.cpu())
        plan = fm.plan_positions(gathered, world, E, fz.SEG_ALIGN)
        fm.check_tiling(plan, gathered, world, E)
        order = torch.argsort(idx.cpu(), dim=1, stable=True)           # the kernel walks sorted picks
        want = plan["pos"][rank].gather(1, order)
        got = p["pos"].cpu().long().view(T, k)
        res = {"pos_equal": bool(torch.equal(got, want)),
               "seg_start_equal": bool(torch.equal(p["seg_start"].cpu().long(), plan["seg_start"][rank])),
               "seg_count_equal": bool(torch.equal(p["seg_count"].cpu().long(), plan["seg_count"][rank])),
               "status": fctx.take_status()}
        dist.barrier()
        if world >= 2:       # two-hop: arrival rows at the representatives against the host model
            ep2 = fctx.next_epoch()
            p2 = fz._plan(fctx, idx, gates, "two_hop", ep2)
            fz._dispatch(fctx, p2, x, "two_hop", ep2)
            torch.cuda.synchronize()
            reps, rows = fm.hop_a_rows(gathered, world, E, 1, 2, fctx.tokens)
            res["rowa_equal"] = bool(torch.equal(p2["rowa"].cpu().long().view(T, 2), rows[rank]))
            res["two_hop_pos_equal"] = bool(torch.equal(p2["pos"].cpu().long().view(T, k), want))
            res["status2"] = fctx.take_status()
            dist.barrier()
        if world == 1:       # every row of this rank's buffer holds the token the model put there
            xin = fctx.section(fz.XIN)
            tok = torch.arange(T).unsqueeze(1).expand(T, k)
            res["rows_equal"] = bool(torch.equal(xin[plan["pos"][0].reshape(-1).to(dev)],
                                                 x[tok.reshape(-1).to(dev)]))
        queue.put((rank, res))
        dist.barrier()
    except Exception as exc:  # noqa: BLE001
        import traceback
        queue.put((rank, "error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2])
def test_fused_positions_match_host_model(native_ops, world):
    """The placement computed by the plan and push kernels equals the host model's arithmetic."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_model_worker, args=(r, world, 29760 + world, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = []
    try:
        for _ in range(world):
            out.append(q.get(timeout=300))
    finally:
        for p in procs:
            p.join(timeout=30)
        for p in procs:
            if p.is_alive():
                p.terminate()
    for item in out:
        assert item[1] != "error", item[2]
        # booleans must be True, status words 0 (False == 0 in Python, so test the type first)
        assert all(v is True if isinstance(v, bool) else v == 0 for v in item[1].values()), item


@pytest.mark.parametrize("world,rpn,n", [(2, 1, 2), (4, 2, 3)])
def test_token_pipeline_keeps_one_hop_two_hop_identity(native_ops, monkeypatch, world, rpn, n):
    """n token slices on n streams and n arenas: the two hops still agree bit for bit; outputs and
    input gradients equal the unsliced remote-read schedule bit for bit, weight gradients within
    rounding."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    monkeypatch.setenv("TERRACE_EP_PIPELINE", str(n))
    _check_ranks(_run(world, 2, 29805 + world, rpn=rpn), world, pipeline=n)
