"""Host model of the fused expert-parallel step: placement tiling, numerics, flag protocol."""
import os

import pytest
import torch

from terracemoe_simulator_b200.parallel import fused_model as fm
from terracemoe_simulator_b200.routing import TRouteConfig, t_route


def _routing(world, T, E, n_groups, k, M, seed):
    cfg = TRouteConfig(E, n_groups, k, M)
    out = []
    for r in range(world):
        g = torch.Generator().manual_seed(seed + r)
        idx, gates, _ = t_route(torch.rand(T + 7 * r, E, generator=g), torch.zeros(E), cfg)
        out.append((idx, gates))
    return cfg, out


@pytest.mark.parametrize("world,E,n_groups,k,M,align", [(4, 16, 4, 4, 2, 64), (8, 64, 4, 6, 2, 64),
                                                      (2, 8, 2, 2, 2, 1), (1, 8, 4, 4, 2, 64)])
def test_positions_tile_every_owner_segment(world, E, n_groups, k, M, align):
    _, routed = _routing(world, 50, E, n_groups, k, M, seed=3)
    idx = [i for i, _ in routed]
    plan = fm.plan_positions(idx, world, E, align)
    fm.check_tiling(plan, idx, world, E)
    epr = E // world
    for o in range(world):
        assert all(int(s) % align == 0 for s in plan["seg_start"][o])
        assert plan["rows"][o] % align == 0
        total = sum(int((i // epr == o).sum()) for i in idx)
        assert int(plan["seg_count"][o].sum()) == total


def test_check_tiling_catches_a_wrong_plan():
    _, routed = _routing(2, 20, 8, 2, 2, 2, seed=1)
    idx = [i for i, _ in routed]
    plan = fm.plan_positions(idx, 2, 8, 64)
    plan["pos"][1][0, 0] = plan["pos"][0][0, 0] if int(plan["owner"][0][0, 0]) == int(
        plan["owner"][1][0, 0]) else plan["pos"][1][0, 0] + 1
    with pytest.raises(AssertionError):
        fm.check_tiling(plan, idx, 2, 8)
    with pytest.raises(ValueError):
        fm.plan_positions([torch.tensor([[1, 1]])], 1, 4)            # an expert picked twice


def test_one_hop_model_matches_the_dense_definition():
    torch.manual_seed(0)
    world, E, H, d = 4, 16, 32, 16
    cfg, routed = _routing(world, 24, E, 4, 4, 2, seed=9)
    w13 = torch.randn(E, H, 2 * d) * H ** -0.5
    w2 = torch.randn(E, d, H) * d ** -0.5
    xs = [torch.randn(i.shape[0], H) for i, _ in routed]
    ys = fm.one_hop_model(xs, [i for i, _ in routed], [g for _, g in routed], w13, w2,
                          cfg.group_size)
    for x, (idx, gates), y in zip(xs, routed, ys):
        ref = torch.zeros_like(x)
        for t in range(x.shape[0]):
            for j in range(idx.shape[1]):
                e = int(idx[t, j])
                a, b = (x[t] @ w13[e]).chunk(2)
                ref[t] += gates[t, j] * ((torch.nn.functional.silu(a) * b) @ w2[e])
        torch.testing.assert_close(y, ref, rtol=1e-4, atol=1e-5)


def test_model_does_not_depend_on_how_tokens_are_split_over_ranks():
    """The same tokens on 1 rank or spread over 4 give the same output rows, bit for bit:
    placement only decides where a row is computed, never what is added to what."""
    torch.manual_seed(1)
    E, H, d = 16, 32, 16
    cfg = TRouteConfig(E, 4, 4, 2)
    x = torch.randn(40, H).bfloat16()
    idx, gates, _ = t_route(torch.rand(40, E), torch.zeros(E), cfg)
    w13 = (torch.randn(E, H, 2 * d) * H ** -0.5).bfloat16()
    w2 = (torch.randn(E, d, H) * d ** -0.5).bfloat16()
    gates = gates.bfloat16()
    whole = fm.one_hop_model([x], [idx], [gates], w13, w2, cfg.group_size)[0]
    parts = fm.one_hop_model(list(x.chunk(4)), list(idx.chunk(4)), list(gates.chunk(4)),
                             w13, w2, cfg.group_size)
    assert torch.equal(torch.cat(parts), whole)


def test_epoch_flags_bounded_wait_and_monotone_epochs():
    flags = fm.EpochFlags(kinds=3, world=4)
    for s in range(4):
        flags.signal(1, s, epoch=5)
    assert flags.wait(1, range(4), epoch=5) == fm.ST_OK
    assert flags.wait(1, range(4), epoch=4) == fm.ST_OK               # older epochs stay satisfied
    flags.signal(1, 2, epoch=3)                                       # a stale signal never lowers
    assert flags.wait(1, range(4), epoch=5) == fm.ST_OK
    # a rank that never signals: the wait gives up with a status instead of blocking
    polls = []
    status = flags.wait(1, range(4), epoch=6, max_polls=50, on_poll=lambda: polls.append(1))
    assert status == fm.ST_TIMEOUT_FLAG and len(polls) == 50
    assert flags.wait(2, [0], epoch=1, max_polls=3, timeout_code=fm.ST_TIMEOUT_COUNTS) \
        == fm.ST_TIMEOUT_COUNTS
    # the late rank arrives during the wait
    late = iter(range(10))
    status = flags.wait(1, range(4), epoch=6, max_polls=50,
                        on_poll=lambda: [flags.signal(1, s, 6) for s in range(4)]
                        if next(late) == 3 else None)
    assert status == fm.ST_OK


@pytest.mark.parametrize("world,E,n_groups,k,M", [(4, 16, 4, 4, 2), (2, 8, 2, 2, 2), (1, 8, 4, 4, 2)])
def test_return_maps_cover_real_rows_once(world, E, n_groups, k, M):
    """Epilogue-push variant: every real row of every owner has exactly one return address,
    padding rows have none, and every (source, slot) is addressed exactly once."""
    _, routed = _routing(world, 40, E, n_groups, k, M, seed=5)
    idx = [i for i, _ in routed]
    plan = fm.plan_positions(idx, world, E, 64)
    slots = max(i.numel() for i in idx)
    maps = fm.return_maps(plan, idx, world, slots)
    seen = set()
    for o in range(world):
        real = torch.zeros_like(maps[o], dtype=torch.bool)
        for a, n in zip(plan["seg_start"][o].tolist(), plan["seg_count"][o].tolist()):
            real[a:a + n] = True
        assert bool(((maps[o] >= 0) == real).all())
        vals = maps[o][real].tolist()
        assert not seen.intersection(vals)
        seen.update(vals)
    want = {s * slots + p for s, i in enumerate(idx) for p in range(i.numel())}
    assert seen == want


def test_epilogue_push_model_equals_pull_model_bitwise():
    torch.manual_seed(1)
    world, E, H, d = 4, 16, 32, 16
    cfg, routed = _routing(world, 24, E, 4, 4, 2, seed=11)
    w13 = (torch.randn(E, H, 2 * d) * H ** -0.5).bfloat16()
    w2 = (torch.randn(E, d, H) * d ** -0.5).bfloat16()
    xs = [torch.randn(i.shape[0], H).bfloat16() for i, _ in routed]
    args = (xs, [i for i, _ in routed], [g for _, g in routed], w13, w2, cfg.group_size)
    pull = fm.one_hop_model(*args)
    push = fm.one_hop_model(*args, epilogue_push=True)
    for a, b in zip(pull, push):
        assert torch.equal(a, b)


def test_scatter_rows_skips_and_counts_bad_addresses():
    yout = [torch.ones(4, 8)]
    maps = [torch.tensor([0, 5, -1, 99])]            # 99 is outside 1 rank x 8 slots
    ret, skipped = fm.scatter_rows(yout, maps, 1, 8, 8, torch.float32)
    assert skipped == 1
    assert ret[0][0].sum() == 8 and ret[0][5].sum() == 8 and ret[0].sum() == 16


class _RecorderLib:
    """Stands in for the native op namespace: records op names, returns tensors of the right
    shapes so that the Python orchestration of ``parallel/fused.py`` can run on a CPU."""

    def __init__(self, T, k, H, epr, cap_rows):
        self.calls, self.T, self.k, self.H, self.epr, self.cap = [], T, k, H, epr, cap_rows
        self.check_schema = False

    @staticmethod
    def _check_schema(name, args):
        """Arguments must fit the registered schema of the real op (count and basic types)."""
        schema = getattr(torch.ops.terrace, name).default._schema
        formal = schema.arguments
        assert len(args) <= len(formal), (name, len(args), len(formal))
        for i, f in enumerate(formal):
            if i >= len(args):
                assert f.has_default_value(), f"{name}: argument {f.name} missing"
                continue
            v, t = args[i], str(f.type)
            if t == "Tensor":
                ok = torch.is_tensor(v)
            elif t == "Optional[Tensor]":
                ok = v is None or torch.is_tensor(v)
            elif t == "int":
                ok = isinstance(v, int) and not isinstance(v, bool)
            elif t == "bool":
                ok = isinstance(v, bool)
            elif t == "float":
                ok = isinstance(v, (int, float)) and not isinstance(v, bool)
            else:
                ok = True
            assert ok, f"{name}: argument {i} ({f.name}: {t}) got {type(v).__name__}"

    def __getattr__(self, name):
        def op(*a, **kw):
            self.calls.append(name)
            assert not kw
            if self.check_schema:
                self._check_schema(name, a)
            T, k, H = self.T, self.k, self.H
            if name in ("ep_plan_pass1",):
                T = a[0].shape[0]
            elif name in ("hopa_push", "hopa_rank", "ep_pull_combine", "origin_combine",
                          "origin_pull_dgate"):
                T = a[1].shape[0]                      # x, es or pos: one row per token
            i32 = dict(dtype=torch.int32)
            if name == "ep_plan_pass1":
                return (torch.zeros(T, k, **i32), torch.zeros(T, k), torch.zeros(T, k, **i32),
                        torch.zeros(T, k, **i32), torch.zeros(128, 16, **i32))
            if name == "ep_plan":
                return (torch.zeros(16, **i32), torch.zeros(self.epr, **i32),
                        torch.zeros(self.epr, **i32), torch.zeros(1, **i32),
                        torch.zeros(16, **i32))
            if name == "hopa_rank":
                return torch.zeros(T, 2, **i32), torch.zeros(128, 2, **i32)
            if name == "hopa_push":
                return torch.zeros(T, k, **i32), torch.zeros(T, 2, **i32)
            if name == "origin_pull_dgate":
                return torch.zeros(T, k)
            if name in ("ep_pull_combine", "origin_combine"):
                return torch.zeros(T, H, dtype=torch.bfloat16)
            if name == "grouped_wgrad":
                return torch.zeros(self.epr, a[0].shape[1], a[1].shape[1], dtype=torch.bfloat16)
            if name == "swiglu_bwd":
                return torch.zeros_like(a[0])
            return None
        return op


def _fake_context(fz, *, T, k, H, d, epr, cap, world, n_nodes, two_hop, overlap, chunks=2):
    """A FusedEPContext with every attribute the orchestration reads and no arena behind it."""
    c = object.__new__(fz.FusedEPContext)
    c.cfg = TRouteConfig(16, 2, 4, 2)
    c.world, c.rank, c.rpn, c.tokens, c.cap_rows, c.epoch = world, 0, 1, T, cap, 0
    c.arena, c.done = torch.zeros(1, dtype=torch.uint8), torch.zeros(8, dtype=torch.int32)
    c.two_hop_ok, c.overlap, c.ret_slots, c.ret2_slots = two_hop, overlap, T * k, n_nodes * T * 2
    c.one_hop_ok = True
    c.E, c.epr, c.k, c.M, c.q, c.hidden, c.d_expert = 16, epr, k, 2, 2, H, d
    c.n_nodes, c.device = n_nodes, torch.device("cpu")
    c.chunks = fz.chunk_ranges(epr, chunks if overlap else 1)
    names = list(fz._BASE_SECTIONS) + ["ret", "dret", "rowmap", "ret2", "dret2"]
    c.off = {n: 256 * i for i, n in enumerate(names)}
    c.ret_base = c.dret_base = c.ret2_base = c.dret2_base = torch.zeros(world, dtype=torch.int64)
    c.row_map = torch.zeros(cap, dtype=torch.int32)
    c.side, c._events, c._inflight = None, [], None
    return c


@pytest.mark.parametrize("overlap", [False, True])
def test_fused_orchestration_launch_sequence(monkeypatch, overlap):
    """Which ops one fused one-hop step issues: the remote-read schedule, and the overlap
    schedule (two chunks of experts, scattering epilogues, local combine)."""
    from terracemoe_simulator_b200.parallel import fused as fz
    T, k, H, d, epr, cap = 8, 4, 32, 16, 16, 128
    rec = _RecorderLib(T, k, H, epr, cap)
    monkeypatch.setenv("TERRACE_CUSTOM_OPS", "1")
    from terracemoe_simulator_b200 import ops
    ops.reset()
    rec.check_schema = ops.status().loaded       # the real schemas, when the library is built
    assert rec.check_schema or not os.path.isfile(ops.status().lib or "")
    monkeypatch.setattr(fz, "_lib", lambda: rec)
    fctx = _fake_context(fz, T=T, k=k, H=H, d=d, epr=epr, cap=cap, world=1, n_nodes=1,
                         two_hop=False, overlap=overlap)
    monkeypatch.setattr(fz.FusedEPContext, "section",
                        lambda self, sel: torch.zeros(cap, H, dtype=torch.bfloat16))
    x = torch.zeros(T, H, dtype=torch.bfloat16, requires_grad=True)
    gates = torch.full((T, k), 0.25, requires_grad=True)
    w13 = torch.zeros(epr, H, 2 * d, dtype=torch.bfloat16, requires_grad=True)
    w2 = torch.zeros(epr, d, H, dtype=torch.bfloat16, requires_grad=True)
    idx = torch.zeros(T, k, dtype=torch.int64)
    y = fz.fused_moe_forward(fctx, x, idx, gates, w13, w2, mode="one_hop")
    fwd = list(rec.calls)
    rec.calls.clear()
    # a second forward while the first waits for its backward would overwrite the arena rows
    with pytest.raises(RuntimeError, match="one forward may be outstanding"):
        fz.fused_moe_forward(fctx, x, idx, gates, w13, w2, mode="one_hop")
    with pytest.raises(RuntimeError, match="one forward may be outstanding"):
        fz.fused_dispatch_combine(fctx, x.detach(), idx, gates.detach(), mode="one_hop")
    assert rec.calls == []
    y.backward(torch.zeros_like(y))
    bwd = list(rec.calls)
    if overlap:
        assert fwd == ["ep_plan_pass1", "ep_plan", "ep_push", "ep_push", "zero_pad_rows",
                       "grouped_gemm_ex", "grouped_gemm_scatter", "grouped_gemm_ex",
                       "grouped_gemm_scatter", "ep_signal", "ep_pull_combine"]
        assert bwd == ["ep_push", "ep_push", "zero_pad_rows", "grouped_gemm_ex",
                       "grouped_wgrad_out", "grouped_gemm_ex", "grouped_wgrad_out",
                       "grouped_wgrad", "grouped_gemm_scatter", "ep_signal", "ep_pull_combine"]
    else:
        assert fwd == ["ep_plan_pass1", "ep_plan", "ep_push", "zero_pad_rows", "grouped_gemm_ex",
                       "grouped_gemm_ex", "ep_signal", "ep_pull_combine"]
        assert bwd == ["ep_push", "zero_pad_rows", "grouped_gemm_ex", "grouped_wgrad",
                       "grouped_wgrad", "grouped_gemm_ex", "ep_signal", "ep_pull_combine"]
    assert x.grad.shape == x.shape and gates.grad.shape == gates.shape
    assert w13.grad.shape == w13.shape and w2.grad.shape == w2.shape
    # the backward released the context: the next forward goes through, and a forward whose
    # graph is dropped without a backward releases it too
    y2 = fz.fused_moe_forward(fctx, x, idx, gates, w13, w2, mode="one_hop")
    del y2
    fz.fused_moe_forward(fctx, x, idx, gates, w13, w2, mode="one_hop")
    monkeypatch.undo()
    ops.reset()


def test_chunk_ranges_and_flag_values():
    from terracemoe_simulator_b200.parallel import fused as fz
    assert fz.chunk_ranges(8, 2) == [(0, 4), (4, 8)]
    assert fz.chunk_ranges(8, 3) == [(0, 3), (3, 6), (6, 8)]
    assert fz.chunk_ranges(2, 4) == [(0, 1), (1, 2)] and fz.chunk_ranges(5, 1) == [(0, 5)]
    # values grow inside a step and from step to step; the last chunk always writes "all"
    vals = [fz.flag_value(ep, i, 3) for ep in (1, 2) for i in range(3)]
    assert vals == sorted(vals) and len(set(vals)) == len(vals)
    assert fz.flag_value(3, 0, 1) == fz.flag_value(3, 7, 8) == 3 * fz.FLAG_STRIDE + 15
    assert fz.flag_value(3, fz.MAX_CHUNKS - 2, fz.MAX_CHUNKS) < fz.flag_value(3, 0, 1)


@pytest.mark.parametrize("overlap", [False, True])
def test_fused_two_hop_orchestration_launch_sequence(monkeypatch, overlap):
    from terracemoe_simulator_b200 import ops
    from terracemoe_simulator_b200.parallel import fused as fz
    T, k, H, d, epr, cap = 8, 4, 32, 16, 8, 128
    rec = _RecorderLib(T, k, H, epr, cap)
    monkeypatch.setenv("TERRACE_CUSTOM_OPS", "1")
    ops.reset()
    rec.check_schema = ops.status().loaded
    monkeypatch.setattr(fz, "_lib", lambda: rec)
    fctx = _fake_context(fz, T=T, k=k, H=H, d=d, epr=epr, cap=cap, world=2, n_nodes=2,
                         two_hop=True, overlap=overlap)
    monkeypatch.setattr(fz.FusedEPContext, "section",
                        lambda self, sel: torch.zeros(cap, H, dtype=torch.bfloat16))
    x = torch.zeros(T, H, dtype=torch.bfloat16, requires_grad=True)
    gates = torch.full((T, k), 0.25, requires_grad=True)
    w13 = torch.zeros(epr, H, 2 * d, dtype=torch.bfloat16, requires_grad=True)
    w2 = torch.zeros(epr, d, H, dtype=torch.bfloat16, requires_grad=True)
    y = fz.fused_moe_forward(fctx, x, torch.zeros(T, k, dtype=torch.int64), gates, w13, w2,
                             mode="two_hop")
    fwd = list(rec.calls)
    rec.calls.clear()
    y.backward(torch.zeros_like(y))
    if overlap:
        assert fwd == ["ep_plan_pass1", "hopa_rank", "ep_plan", "hopa_push", "arrival_push",
                       "arrival_push", "zero_pad_rows", "grouped_gemm_ex", "grouped_gemm_scatter",
                       "grouped_gemm_ex", "grouped_gemm_scatter", "ep_signal", "arrival_combine",
                       "origin_combine"]
        assert rec.calls == ["hopa_push", "arrival_push", "arrival_push", "zero_pad_rows",
                             "grouped_gemm_ex", "grouped_wgrad_out", "grouped_gemm_ex",
                             "grouped_wgrad_out", "grouped_wgrad", "grouped_gemm_scatter", "ep_signal", "arrival_combine",
                             "origin_combine", "origin_pull_dgate"]
    else:
        assert fwd == ["ep_plan_pass1", "hopa_rank", "ep_plan", "hopa_push", "arrival_push",
                       "zero_pad_rows", "grouped_gemm_ex", "grouped_gemm_ex", "ep_signal",
                       "arrival_combine", "origin_combine"]
        assert rec.calls == ["hopa_push", "arrival_push", "zero_pad_rows", "grouped_gemm_ex",
                             "grouped_wgrad", "grouped_wgrad", "grouped_gemm_ex", "ep_signal",
                             "arrival_combine", "origin_combine", "origin_pull_dgate"]
    assert gates.grad.shape == gates.shape
    monkeypatch.undo()
    ops.reset()


def test_capacity_in_the_plan_keeps_exactly_the_picks_apply_capacity_keeps():
    """The device-side cap (canonical order: source rank, then token) against the layer-level
    oracle ``apply_capacity`` with the lower ranks' counts as ``prior_counts``."""
    from terracemoe_simulator_b200.layer import apply_capacity
    from terracemoe_simulator_b200.parallel.fused import expert_capacity
    world, E, k = 4, 16, 4
    cfg, routed = _routing(world, 40, E, 4, k, 2, seed=31)
    idx = [i for i, _ in routed]
    tokens_global = sum(i.shape[0] for i in idx)
    cap = expert_capacity(0.6, tokens_global, k, E)
    plan = fm.plan_positions(idx, world, E, 64, cap=cap)
    counts = torch.stack([torch.bincount(i.reshape(-1), minlength=E) for i in idx])
    dropped = 0
    for s in range(world):
        prior = counts[:s].sum(0)
        _, keep, cap_ref = apply_capacity(idx[s], routed[s][1], E, 0.6,
                                          n_tokens_global=tokens_global, prior_counts=prior)
        assert cap_ref == cap
        assert torch.equal(plan["pos"][s] >= 0, keep)
        dropped += int((~keep).sum())
    assert dropped > 0                                    # the factor really binds
    for o in range(world):
        assert int(plan["seg_count"][o].max()) <= cap
    # kept rows still tile every (shrunk) segment exactly once
    kept_idx = [i.clone() for i in idx]
    taken = [torch.zeros(max(plan["rows"][o], 1), dtype=torch.int64) for o in range(world)]
    for s in range(world):
        live = plan["pos"][s] >= 0
        for o in range(world):
            rows = plan["pos"][s][live & (plan["owner"][s] == o)]
            taken[o].scatter_add_(0, rows, torch.ones_like(rows))
    epr = E // world
    for o in range(world):
        assert int(taken[o].max()) <= 1
        for le in range(epr):
            a, n = int(plan["seg_start"][o][le]), int(plan["seg_count"][o][le])
            assert bool((taken[o][a:a + n] == 1).all())
    del kept_idx


def test_single_mode_contexts_shrink_the_other_paths_sections():
    """The decoder benchmark's layer (32768 tokens per GPU, top-4, width 2048, 8 GPUs in groups of
    2): a context built for one path carries about half the bytes of one built for both."""
    from terracemoe_simulator_b200.parallel import fused as fz
    T, k, q, H, world, n_nodes = 32768, 4, 2, 2048, 8, 4
    cap_rows = 2 * T * k

    def total(one_hop, two_hop):
        sizes = fz.section_sizes(world=world, n_experts=64, hidden=H, q=q, cap_rows=cap_rows,
                                 arrival_rows=n_nodes * T if two_hop else 1, out_rows=1,
                                 overlap=True, own_slots=T * k if one_hop else 1,
                                 rep_slots=n_nodes * T * q if two_hop else 1)
        assert list(sizes)[:12] == list(fz._BASE_SECTIONS)
        return fz.arena_layout(list(sizes.values()))[2]
    both, one, two = total(True, True), total(True, False), total(False, True)
    assert one < 0.5 * both and two < 0.9 * both
    assert one == pytest.approx((2 * cap_rows + 2 * T * k) * H * 2, rel=0.01)
    ctx = _fake_context(fz, T=8, k=4, H=32, d=16, epr=16, cap=128, world=2, n_nodes=2,
                        two_hop=True, overlap=True)
    ctx.one_hop_ok = False
    with pytest.raises(ValueError, match="built for two_hop only"):
        ctx.check_mode("one_hop")
    ctx.check_mode("two_hop")


@pytest.mark.parametrize("T", [7, 300, 900, 5000])
def test_first_plan_pass_ranks_picks_in_token_order(T):
    """The ranking the plan kernel computes per chunk, replayed on the host: with distinct
    experts per token the position of a pick inside its expert is the number of earlier tokens
    that picked it -- the order the capacity rule and ``plan_positions`` assume; with a repeated
    expert the ranks are still a permutation inside every expert."""
    from terracemoe_simulator_b200.parallel import fused_model as fm
    g = torch.Generator().manual_seed(T)
    E, k = 16, 4
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    es, rank_local, hist = fm.pass1_ranks(idx, E)
    per = -(-T // 128)
    base = torch.cumsum(hist, 0) - hist
    chunk = (torch.arange(T) // per).unsqueeze(1).expand(T, k)
    within = base[chunk, es] + rank_local
    onehot = torch.zeros(T, E, dtype=torch.long).scatter_add_(1, idx, torch.ones_like(idx))
    earlier = torch.cumsum(onehot, 0) - onehot
    assert torch.equal(within, earlier.gather(1, es))
    assert torch.equal(hist.sum(0), torch.bincount(idx.reshape(-1), minlength=E))
    # the placement model built on the same order
    plan = fm.plan_positions([idx], 1, E, seg_align=1)
    assert torch.equal(plan["pos"][0].gather(1, torch.argsort(idx, dim=1, stable=True)),
                       plan["seg_start"][0][es] + within)
    dup = torch.randint(0, E, (T, k), generator=g)
    es2, ranks2, hist2 = fm.pass1_ranks(dup, E)
    within2 = (torch.cumsum(hist2, 0) - hist2)[chunk, es2] + ranks2
    for e in range(E):
        got = torch.sort(within2[es2 == e]).values
        assert torch.equal(got, torch.arange(got.numel()))


def test_arena_layout_puts_a_guard_after_every_section():
    from terracemoe_simulator_b200.parallel.fused import GUARD_BYTES, arena_layout
    sizes = [100, 4096, 1, 256 * 7 + 3]
    offs, guards, total = arena_layout(sizes)
    assert offs[0] == 0 and all(o % 256 == 0 for o in offs + guards)
    for i, s in enumerate(sizes):
        assert offs[i] + s <= guards[i]                          # the section ends before its guard
        end = offs[i + 1] if i + 1 < len(sizes) else total
        assert guards[i] + GUARD_BYTES <= end                    # and the guard before the next
    assert arena_layout(sizes, guard=0)[2] == sum((s + 255) // 256 * 256 for s in sizes)


@pytest.mark.parametrize("world,rpn,E,k,M", [(4, 1, 16, 4, 2), (8, 2, 32, 6, 2), (4, 2, 16, 4, 2)])
def test_two_hop_model_equals_one_hop_model_bitwise(world, rpn, E, k, M):
    """The claim the GPU tests check on hardware, restated on the host: with origin-computed
    positions and the canonical reduction tree the two paths give the same bits."""
    torch.manual_seed(2)
    n_groups = world // rpn
    cfg, routed = _routing(world, 12, E, n_groups, k, M, seed=21)
    H, d = 32, 16
    w13 = (torch.randn(E, H, 2 * d) * H ** -0.5).bfloat16()
    w2 = (torch.randn(E, d, H) * d ** -0.5).bfloat16()
    xs = [torch.randn(i.shape[0], H).bfloat16() for i, _ in routed]
    idx, gates = [i for i, _ in routed], [g for _, g in routed]
    one = fm.one_hop_model(xs, idx, gates, w13, w2, cfg.group_size)
    two = fm.two_hop_model(xs, idx, gates, w13, w2, rpn, M)
    for a, b in zip(one, two):
        assert torch.equal(a, b)


def test_hop_a_rows_fill_each_source_block_from_zero_without_gaps():
    world, rpn, E, k, M = 8, 2, 32, 6, 2
    _, routed = _routing(world, 20, E, world // rpn, k, M, seed=4)
    idx = [i for i, _ in routed]
    cap = max(i.shape[0] for i in idx)
    reps, rows = fm.hop_a_rows(idx, world, E, rpn, M, cap)
    for s in range(world):
        assert bool((reps[s] % rpn == s % rpn).all())                # same local index as the source
        block = rows[s] // cap
        assert bool((block == s // rpn).all())                       # the source group's block
        for g in range(world // rpn):
            mine = (reps[s] // rpn == g)
            got = sorted((rows[s][mine] % cap).tolist())
            assert got == list(range(len(got)))                      # ranks 0 .. n-1, each once
    with pytest.raises(ValueError):                                  # global top-k is not quota-shaped
        bad = [torch.tensor([[0, 1, 2, 9, 17, 25]])] * world
        fm.hop_a_rows(bad, world, E, rpn, M, cap)


def test_push_back_rows_are_distinct_slots_of_the_origin_section():
    world, rpn, E, k, M = 8, 2, 32, 6, 2
    _, routed = _routing(world, 20, E, world // rpn, k, M, seed=6)
    idx = [i for i, _ in routed]
    cap = max(i.shape[0] for i in idx)
    reps, rows = fm.hop_a_rows(idx, world, E, rpn, M, cap)
    for s in range(world):
        local = fm.push_back_rows(rows[s], reps[s], rpn, cap)
        assert int(local.min()) >= 0 and int(local.max()) < (world // rpn) * cap
        assert local.unique().numel() == local.numel()               # one slot per (token, group)
        assert bool((local // cap == reps[s] // rpn).all())          # block of the sending group


def test_pipelined_context_slices_tokens_and_runs_every_slice(monkeypatch):
    """The token-sliced pipeline: each slice runs the unsliced op sequence on its own context;
    outputs come back in token order (CPU: no streams, the recorder stands in for the kernels)."""
    from terracemoe_simulator_b200 import ops
    from terracemoe_simulator_b200.parallel import fused as fz
    T, k, H, d, epr, cap = 10, 4, 32, 16, 16, 128

    rec = _RecorderLib(T, k, H, epr, cap)
    monkeypatch.setenv("TERRACE_CUSTOM_OPS", "1")
    ops.reset()
    rec.check_schema = ops.status().loaded
    monkeypatch.setattr(fz, "_lib", lambda: rec)

    def fake_ctx(tokens):
        return _fake_context(fz, T=tokens, k=k, H=H, d=d, epr=epr, cap=cap, world=1, n_nodes=1,
                             two_hop=False, overlap=False)

    monkeypatch.setattr(fz.FusedEPContext, "section",
                        lambda self, sel: torch.zeros(cap, H, dtype=torch.bfloat16))
    pipe = object.__new__(fz.PipelinedFusedEP)
    pipe.n, pipe.tokens, pipe.slice_tokens = 3, T, 4
    pipe.ctxs, pipe.streams = [fake_ctx(4) for _ in range(3)], [None] * 3
    pipe.device, pipe.two_hop_ok = torch.device("cpu"), False
    assert pipe.bounds(10) == [(0, 4), (4, 8), (8, 10)] and pipe.bounds(3) == [(0, 1), (1, 2), (2, 3)]
    x = torch.zeros(T, H, dtype=torch.bfloat16, requires_grad=True)
    gates = torch.full((T, k), 0.25, requires_grad=True)
    w13 = torch.zeros(epr, H, 2 * d, dtype=torch.bfloat16, requires_grad=True)
    w2 = torch.zeros(epr, d, H, dtype=torch.bfloat16, requires_grad=True)
    y = fz.run_fused(pipe, x, torch.zeros(T, k, dtype=torch.int64), gates, w13, w2, mode="one_hop")
    assert y.shape == (T, H)
    assert rec.calls.count("ep_push") == 3 and rec.calls.count("ep_pull_combine") == 3
    assert [c.epoch for c in pipe.ctxs] == [1, 1, 1]
    y.backward(torch.zeros_like(y))
    assert x.grad.shape == x.shape and w13.grad.shape == w13.shape
    with pytest.raises(ValueError):
        fz.run_fused(pipe, torch.zeros(T + 1, H, dtype=torch.bfloat16),
                     torch.zeros(T + 1, k, dtype=torch.int64), torch.zeros(T + 1, k), w13, w2,
                     mode="one_hop")
    monkeypatch.setenv("TERRACE_EP_PIPELINE", "2")
    assert fz.pipeline_depth() == 2
    monkeypatch.setenv("TERRACE_EP_PIPELINE", "9")
    with pytest.raises(ValueError):
        fz.pipeline_depth()
    monkeypatch.undo()
    ops.reset()


def test_canary_check_flags_the_section_whose_guard_was_overwritten():
    from terracemoe_simulator_b200.parallel.fused import (GUARD_BYTES, GUARD_VALUE, FusedEPContext,
                                                          arena_layout)
    sizes = [100, 4096, 1, 256 * 7 + 3]
    offs, guards, total = arena_layout(sizes)
    c = object.__new__(FusedEPContext)
    c.buf, c.guards = torch.zeros(total, dtype=torch.uint8), guards
    c._guard_index = torch.tensor(guards, dtype=torch.int64).unsqueeze(1) + torch.arange(GUARD_BYTES)
    c.buf[c._guard_index.reshape(-1)] = GUARD_VALUE
    assert c.check_canaries() == []
    c.buf[offs[1]:offs[1] + 4096] = 7                  # filling a whole section touches no guard
    assert c.check_canaries() == []
    c.buf[offs[2] + 256 + 5] = 0                       # one byte past the padded end of section 2
    assert c.check_canaries() == [2]
