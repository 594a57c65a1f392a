"""Fake cluster: 4 gloo processes = 2 groups of 2 ranks, so the cross-group hop is real (CPU).

One spawn per scenario set; every rank returns its tensors through a queue and the parent
asserts.  Canonical geometry: world 4, rpn 2, 16 experts, k = 4.
"""
import datetime
import os
import traceback

import pytest
import torch
import torch.multiprocessing as mp

WORLD, RPN, E, K, H, D, T = 4, 2, 16, 4, 24, 16, 37


def _np(obj):
    """Tensors -> numpy so that queue items are pickled by value (the child may exit first)."""
    if torch.is_tensor(obj):
        return ("__t__", obj.detach().cpu().numpy())
    if isinstance(obj, dict):
        return {k: _np(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_np(v) for v in obj]
    return obj


def _th(obj):
    if isinstance(obj, list) and len(obj) == 2 and obj[0] == "__t__":
        return torch.from_numpy(obj[1])
    if isinstance(obj, tuple) and len(obj) == 2 and obj[0] == "__t__":
        return torch.from_numpy(obj[1])
    if isinstance(obj, dict):
        return {k: _th(v) for k, v in obj.items()}
    if isinstance(obj, list):
        return [_th(v) for v in obj]
    return obj


def _setup(rank, port, timeout_s=120):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD,
                            timeout=datetime.timedelta(seconds=timeout_s))
    return dist


def _problem(rank, M, dtype=torch.float32):
    from terracemoe_simulator_b200.routing import TRouteConfig, t_route
    g = torch.Generator().manual_seed(0)
    w13 = torch.randn(E, H, 2 * D, generator=g) * H ** -0.5
    w2 = torch.randn(E, D, H, generator=g) * D ** -0.5
    wr = torch.randn(E, H, generator=g) * 0.5
    gx = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(T + rank, H, generator=gx)
    gy = torch.randn(T + rank, H, generator=gx)
    cfg = TRouteConfig(E, WORLD // RPN, K, M)
    return cfg, w13.to(dtype), w2.to(dtype), wr, x.to(dtype), gy.to(dtype), t_route


def _parity_worker(rank, port, queue, M):
    try:
        dist = _setup(rank, port)
        from terracemoe_simulator_b200.parallel import ep
        from terracemoe_simulator_b200.parallel.ep import ep_moe_forward
        from terracemoe_simulator_b200.parallel.ta2a import init_ta2a_groups, ta2a_moe_forward
        init_ta2a_groups(WORLD, RPN)
        cfg, w13, w2, wr, x0, gy, t_route = _problem(rank, M)
        epr = E // WORLD
        out = {}
        counts = {}
        for name in ("one", "two", "two_general", "one_flat"):
            x = x0.clone().requires_grad_(True)
            w = wr.clone().requires_grad_(True)
            a = w13[rank * epr:(rank + 1) * epr].clone().requires_grad_(True)
            b = w2[rank * epr:(rank + 1) * epr].clone().requires_grad_(True)
            idx, gates, _ = t_route(torch.sigmoid(x @ w.t()), torch.zeros(E), cfg)
            before = ep.CALLS["a2a"]
            if name == "one":
                y = ep_moe_forward(x, idx, gates, a, b, WORLD, E, rpn=RPN)
            elif name == "one_flat":
                y = ep_moe_forward(x, idx, gates, a, b, WORLD, E, canonical=False)
            elif name == "two":
                y = ta2a_moe_forward(x, idx, gates, a, b, WORLD, E, rpn=RPN, groups_m=M)
            else:
                y = ta2a_moe_forward(x, idx, gates, a, b, WORLD, E, rpn=RPN, groups_m=None)
            fwd = ep.CALLS["a2a"] - before
            (y * gy).sum().backward()
            counts[name] = (fwd, ep.CALLS["a2a"] - before - fwd)
            out[name] = [t.detach().clone() for t in (y, x.grad, w.grad, a.grad, b.grad)]
        # single-process oracle for this rank's tokens (all experts local)
        x = x0.clone().requires_grad_(True)
        w = wr.clone().requires_grad_(True)
        idx, gates, _ = t_route(torch.sigmoid(x @ w.t()), torch.zeros(E), cfg)
        y = torch.zeros_like(x)
        for e in range(E):
            tok, col = (idx == e).nonzero(as_tuple=True)
            u, v = (x[tok] @ w13[e]).chunk(2, -1)
            y = y.index_add(0, tok, gates[tok, col, None] * ((torch.nn.functional.silu(u) * v) @ w2[e]))
        (y * gy).sum().backward()
        out["oracle"] = [y.detach(), x.grad, w.grad]
        queue.put((rank, _np(out), counts, None))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:                                  # noqa: BLE001
        queue.put((rank, None, None, traceback.format_exc()))


def _spawn(target, args, n=WORLD, timeout=300):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=target, args=(r,) + args[:1] + (q,) + args[1:]) for r in range(n)]
    for p in procs:
        p.start()
    res = [q.get(timeout=timeout) for _ in range(n)]
    for p in procs:
        p.join(timeout=60)
    res = [tuple(_th(v) for v in r) for r in res]
    return sorted(res, key=lambda r: r[0])


@pytest.fixture(scope="module", params=[2, 1])
def parity(request):
    res = _spawn(_parity_worker, (29400 + request.param, request.param))
    for r in res:
        assert r[-1] is None, r[-1]
    return res


def test_one_hop_equals_two_hop_bitwise(parity):
    for rank, out, counts, _ in parity:
        for a, b in zip(out["one"], out["two"]):
            assert torch.equal(a, b)


def test_general_bitmask_path_equals_quota_path(parity):
    for rank, out, counts, _ in parity:
        for a, b in zip(out["two"], out["two_general"]):
            assert torch.equal(a, b)


def test_matches_single_process_oracle_and_reference_order(parity):
    for rank, out, counts, _ in parity:
        for a, b in zip(out["one"][:3], out["oracle"]):
            torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-4)
        for a, b in zip(out["one_flat"], out["one"]):
            torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)


def test_collective_counts_are_pinned(parity):
    for rank, out, counts, _ in parity:
        assert counts["one"] == (4, 2)
        assert counts["two"] == (9, 5)


# ---- seams --------------------------------------------------------------------------------------
def _seam_worker(rank, port, queue):
    try:
        dist = _setup(rank, port)
        from terracemoe_simulator_b200.parallel import pack, seams
        from terracemoe_simulator_b200.parallel.ta2a import (get_ta2a_groups, init_ta2a_groups,
                                                             ta2a_moe_forward)
        from terracemoe_simulator_b200.parallel.ep import swiglu_experts
        init_ta2a_groups(WORLD, RPN)
        intra, inter = get_ta2a_groups(WORLD, RPN)
        M = 2
        cfg, w13, w2, wr, x0, gy, t_route = _problem(rank, M)
        epr = E // WORLD
        a0, b0 = w13[rank * epr:(rank + 1) * epr], w2[rank * epr:(rank + 1) * epr]

        def run(variant, inter_group=None, overlap=False):
            os.environ.pop("TERRACE_TA2A_PACK", None)
            os.environ.pop("TERRACE_TA2A_ASYNC_COUNTS", None)
            os.environ.pop("TERRACE_TA2A_EARLY_HOPB", None)
            if variant in ("off", "small", "full"):
                os.environ["TERRACE_TA2A_PACK"] = variant
            if variant == "sync":
                os.environ["TERRACE_TA2A_ASYNC_COUNTS"] = "0"
                os.environ["TERRACE_TA2A_EARLY_HOPB"] = "0"
            pack.reset()
            seams.reset_async_counts()
            seams.reset_early_hopb()
            x = x0.clone().requires_grad_(True)
            w = wr.clone().requires_grad_(True)
            a, b = a0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
            idx, gates, _ = t_route(torch.sigmoid(x @ w.t()), torch.zeros(E), cfg)
            rmap = torch.zeros(x.shape[0], E, dtype=torch.bool)
            rmap[torch.arange(x.shape[0]).unsqueeze(1), idx] = True
            probs = torch.zeros(x.shape[0], E).index_put(
                (torch.arange(x.shape[0]).unsqueeze(1).expand_as(idx), idx), gates)
            kw = dict(world=WORLD, rank=rank, rpn=RPN, n_experts=E, intra_group=intra,
                      inter_group=inter_group, groups_m=M)
            if overlap:
                saved = []
                permuted, tpe, pprobs, shared, st = seams.ta2a_permute_overlap(
                    x, probs, rmap, save_tensors=saved,
                    run_shared_experts=lambda: x.detach() * 2, **kw)
                assert len(saved) == 7 and torch.equal(shared, x.detach() * 2)
            else:
                permuted, tpe, pprobs, st = seams.ta2a_permute(x, probs, rmap, **kw)
            if overlap:
                # the layer owns the backward: every segment is replayed by hand and the
                # gradients cross Hop A through raw exchanges, outside autograd
                from terracemoe_simulator_b200.parallel.ep import _a2a_raw
                d_in = permuted.detach().requires_grad_(True)
                p_in = pprobs.detach().requires_grad_(True)
                eo = swiglu_experts(d_in, a, b, tpe) * p_in.unsqueeze(-1)
                y = seams.ta2a_unpermute_overlap(eo, st, saved, out_shape=x.shape)
                assert len(saved) == 10 and saved[2] is None
                p1g, p1p, _, p2in, p2g, p2pd, p2pg, u1in, u1g, u2in = saved
                (y * gy).sum().backward()                                   # y <- back_d
                u1g.backward(_a2a_raw(u2in.grad, st.send_l, st.recv_l))     # red <- eo_d
                eo.backward(u1in.grad)                                      # experts
                p2pg.backward(p_in.grad)                                    # gates of stage 2
                d_gate = _a2a_raw(p2pd.grad, st.recv_l, st.send_l)
                p2g.backward(d_in.grad)                                     # rows of stage 2
                d_rows = _a2a_raw(p2in.grad, st.recv_l, st.send_l)
                torch.autograd.backward([p1g, p1p], grad_tensors=[d_rows, d_gate])
            else:
                eo = swiglu_experts(permuted, a, b, tpe) * pprobs.unsqueeze(-1)
                y = seams.ta2a_unpermute(eo, st, x)
                (y * gy).sum().backward()
            return [t.detach().clone() for t in (y, x.grad, w.grad, a.grad, b.grad, tpe)]

        out = {v: run(v) for v in ("small", "off", "full", "sync")}
        out["subgroup"] = run("small", inter_group=inter)
        out["overlap"] = run("small", overlap=True)
        x = x0.clone().requires_grad_(True)
        w = wr.clone().requires_grad_(True)
        a, b = a0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
        idx, gates, _ = t_route(torch.sigmoid(x @ w.t()), torch.zeros(E), cfg)
        y = ta2a_moe_forward(x, idx, gates, a, b, WORLD, E, rpn=RPN, groups_m=M, canonical=False)
        (y * gy).sum().backward()
        out["closed"] = [t.detach().clone() for t in (y, x.grad, w.grad, a.grad, b.grad)]
        live = dict(seams.SEAM_CALLS)
        live.update(pack.PACK_CALLS)
        queue.put((rank, _np(out), live, None))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:                                  # noqa: BLE001
        queue.put((rank, None, None, traceback.format_exc()))


@pytest.fixture(scope="module")
def seam_results():
    res = _spawn(_seam_worker, (29411,))
    for r in res:
        assert r[-1] is None, r[-1]
    return res


def test_seam_variants_are_bitwise_identical(seam_results):
    for rank, out, live, _ in seam_results:
        for variant in ("off", "full", "sync", "subgroup", "overlap"):
            for a, b in zip(out["small"], out[variant]):
                assert torch.equal(a, b), variant


def test_seam_matches_closed_forward(seam_results):
    for rank, out, live, _ in seam_results:
        for a, b in zip(out["small"][:5], out["closed"]):
            torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)


def test_seam_live_path_counters(seam_results):
    for rank, out, live, _ in seam_results:
        assert live["permute"] == 5 and live["permute_overlap"] == 1
        assert live["hopa_small"] >= 3 and live["hopa_full"] >= 1 and live["hopb_meta"] >= 4
        assert live["async_counts"] >= 4 and live["early_hopb"] >= 4


# ---- failure detection on the host --------------------------------------------------------------
def _failure_worker(rank, port, queue):
    try:
        dist = _setup(rank, port, timeout_s=8)
        from terracemoe_simulator_b200.parallel.ep import ep_moe_forward
        cfg, w13, w2, wr, x, gy, t_route = _problem(rank, 2)
        if rank == 3:                  # this rank leaves between steps and never joins the exchange
            queue.put((rank, "left", None))
            return
        idx, gates, _ = t_route(torch.sigmoid(x @ wr.t()), torch.zeros(E), cfg)
        epr = E // WORLD
        try:
            ep_moe_forward(x, idx, gates, w13[rank * epr:(rank + 1) * epr],
                           w2[rank * epr:(rank + 1) * epr], WORLD, E)
            queue.put((rank, "completed", None))
        except Exception as exc:                       # noqa: BLE001
            queue.put((rank, "error", type(exc).__name__))
    except Exception:                                  # noqa: BLE001
        queue.put((rank, "crash", traceback.format_exc()))


def test_missing_rank_surfaces_as_error_not_hang():
    res = _spawn(_failure_worker, (29421,), timeout=120)
    states = {r[0]: r[1] for r in res}
    assert states[3] == "left"
    assert all(states[r] == "error" for r in (0, 1, 2)), res
