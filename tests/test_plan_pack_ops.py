"""Send plan guards, wire formats, packing containers, executable op specs, loader gate (CPU)."""
import logging

import pytest
import torch

from terracemoe_simulator_b200 import ops
from terracemoe_simulator_b200.ops.refs import (fixed_hist, k1_arrival_ref, k2_pack_ref,
                                                stable_bucket_order)
from terracemoe_simulator_b200.parallel import pack
from terracemoe_simulator_b200.parallel.plan import dispatch_stats, plan_ta2a, reset_plan_cache
from terracemoe_simulator_b200.parallel.ta2a import build_expansion, pack_quota_wire
from terracemoe_simulator_b200.routing import TRouteConfig, t_route


def _quota_routing(T, E, n_nodes, k, M, seed=0, sort_rows=True):
    g = torch.Generator().manual_seed(seed)
    per, q = E // n_nodes, k // M
    rows = []
    for _ in range(T):
        groups = torch.randperm(n_nodes, generator=g)[:M]
        picks = torch.cat([grp * per + torch.randperm(per, generator=g)[:q] for grp in groups])
        picks = picks[torch.randperm(k, generator=g)]
        rows.append(picks.sort().values if sort_rows else picks)
    return torch.stack(rows)


# ---- plan ---------------------------------------------------------------------------------------
def test_plan_rows_are_group_major_and_inverse_is_consistent():
    reset_plan_cache()
    world, rpn, E, T, k, M = 8, 2, 32, 40, 4, 2
    idx = _quota_routing(T, E, world // rpn, k, M, 1)
    u_src, u_node, counts, inverse = plan_ta2a(idx, world, E, rpn, groups_m=M)
    assert u_src.shape == (T * M,) and int(counts.sum()) == T * M
    assert torch.all(u_node[1:] >= u_node[:-1])
    for g in range(world // rpn):
        seg = u_src[u_node == g]
        assert torch.all(seg[1:] > seg[:-1])
    slots = (E // world) * rpn
    dest = idx // slots
    assert torch.equal(u_node[inverse].view(T, k), dest)
    assert torch.equal(u_src[inverse].view(T, k), torch.arange(T).unsqueeze(1).expand(T, k))
    general = plan_ta2a(idx, world, E, rpn, groups_m=None)
    for a, b in zip((u_src, u_node, counts, inverse), general):
        assert torch.equal(a, b)


def test_plan_refuses_wrong_fanout_quota_and_divisibility():
    reset_plan_cache()
    world, rpn, E = 4, 2, 8          # 2 groups of 4 experts
    good = torch.tensor([[0, 1, 4, 5], [2, 3, 6, 7]])
    plan_ta2a(good, world, E, rpn, groups_m=2)
    reset_plan_cache()
    one_group = torch.tensor([[0, 1, 2, 3], [4, 5, 6, 7]])
    with pytest.raises(ValueError, match="fan-out"):
        plan_ta2a(one_group, world, E, rpn, groups_m=2)
    reset_plan_cache()
    three_one = torch.tensor([[0, 1, 2, 4], [4, 5, 6, 0]])
    with pytest.raises(ValueError, match="quota"):
        plan_ta2a(three_one, world, E, rpn, groups_m=2)
    with pytest.raises(ValueError, match="divide"):
        plan_ta2a(good, world, E, rpn, groups_m=3)


def test_group_limited_router_output_is_refused_by_the_fast_path():
    reset_plan_cache()
    cfg = TRouteConfig(32, 4, 4, 2)
    aff = torch.rand(512, 32, generator=torch.Generator().manual_seed(2))
    idx, _, _ = t_route(aff, torch.zeros(32), cfg, "group_limited")
    with pytest.raises(ValueError):
        plan_ta2a(idx, 8, 32, 2, groups_m=2)
    reset_plan_cache()
    idx_full, _, _ = t_route(aff, torch.zeros(32), cfg, "full")
    plan_ta2a(idx_full, 8, 32, 2, groups_m=2)


def test_verification_cadence(monkeypatch):
    from terracemoe_simulator_b200.parallel import plan as plan_mod
    reset_plan_cache()
    calls = []
    real = plan_mod._verify_quota
    monkeypatch.setattr(plan_mod, "_verify_quota", lambda *a: (calls.append(1), real(*a)))
    idx = _quota_routing(16, 8, 2, 4, 2, 3)
    for _ in range(plan_mod.VERIFY_EVERY + 2):
        plan_ta2a(idx, 4, 8, 2, groups_m=2)
    assert len(calls) == 2            # first call and the 256th re-verification


def test_dispatch_stats_ledger():
    idx = _quota_routing(64, 32, 4, 6, 2, 4)
    s = dispatch_stats(idx, 8, 32, 2)
    assert s["rows_baseline"] == 64 * 6 and s["rows_ta2a"] == 64 * 2
    assert s["dedup_x"] == 3.0 and s["msgs_baseline"] == 8 and s["msgs_ta2a"] == 4
    assert s["msg_growth_x"] == 2


def test_quota_wire_equals_bitmask_expansion():
    world, rpn, E, T, k, M = 8, 2, 32, 30, 6, 2
    idx = _quota_routing(T, E, 4, k, M, 5)
    gates = torch.rand(T, k, generator=torch.Generator().manual_seed(6))
    u_src, _, _, inverse = plan_ta2a(idx, world, E, rpn, groups_m=M)
    slots, q = (E // world) * rpn, k // M
    slot_tab, gate_tab, rows_tm = pack_quota_wire(idx, gates, inverse, T * M, slots, q)
    mask = build_expansion(idx, inverse, T * M, world, E, rpn)
    assert torch.equal((torch.ones_like(slot_tab) << slot_tab).sum(1), mask)
    assert torch.all(slot_tab[:, 1:] > slot_tab[:, :-1])
    assert torch.equal(u_src[rows_tm], torch.arange(T).unsqueeze(1).expand(T, M))
    with pytest.raises(ValueError):
        build_expansion(idx, inverse, T * M, 2, 256, 2)      # 256 slots: no bitmask


# ---- packing ------------------------------------------------------------------------------------
PACK_GEOMS = [(5, 6, 2, 2), (5, 6, 4, 1), (1, 7, 3, 3), (17, 2048, 3, 3), (4, 5, 1, 1),
              (3, 24, 24, 1), (9, 2048, 24, 1)]


@pytest.mark.parametrize("n,hidden,gate_w,id_w", PACK_GEOMS)
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
def test_hopa_pack_round_trip_bitwise(n, hidden, gate_w, id_w, dt):
    g = torch.Generator().manual_seed(n + hidden)
    payload = torch.randn(n, hidden, generator=g).to(dt)
    gates = torch.rand(n, gate_w, generator=g).to(dt)
    ids = torch.randint(-2 ** 62, 2 ** 62, (n, id_w), generator=g)
    buf, lay = pack.hopa_pack(payload, gates, ids)
    assert buf.dtype == torch.int64 and buf.shape == (n, lay.words)
    p2, g2, i2 = pack.hopa_unpack(buf, lay)
    assert torch.equal(p2, payload) and torch.equal(g2, gates) and torch.equal(i2, ids)
    pack.assert_not_aliased(buf, p2, g2, i2)
    sbuf, slay = pack.hopa_pack_small(gates, ids[:, 0])
    g3, i3 = pack.hopa_unpack_small(sbuf, slay)
    assert torch.equal(g3, gates) and torch.equal(i3, ids[:, 0]) and i3.dim() == 1
    used = slay.id_w * 8 + slay.gate_bytes
    assert torch.all(sbuf.view(torch.uint8).view(n, -1)[:, used:] == 0)      # zero padding
    buf.untyped_storage().resize_(0)
    assert torch.equal(p2, payload)                                         # planes own storage


def test_pack_checks_and_meta():
    with pytest.raises(TypeError):
        pack.hopa_pack(torch.zeros(2, 4), torch.zeros(2, 2, dtype=torch.bfloat16),
                       torch.zeros(2, dtype=torch.int64))
    with pytest.raises(TypeError):
        pack.hopa_pack_small(torch.zeros(2, 2), torch.zeros(2, dtype=torch.int32))
    slot = torch.tensor([3, 0, 62], dtype=torch.int64)
    gate = torch.tensor([0.25, 0.5, 1.0], dtype=torch.bfloat16)
    meta = pack.hopb_pack_meta(slot, gate)
    assert meta.shape == (3, pack.hopb_meta_words())
    s2, g2 = pack.hopb_unpack_meta(meta, torch.bfloat16)
    assert torch.equal(s2, slot) and torch.equal(g2, gate)
    with pytest.raises(AssertionError):
        pack.assert_not_aliased(meta, meta[:, 0])


def test_pack_mode_switch(monkeypatch):
    for value, want in [(None, "small"), ("0", "off"), ("off", "off"), ("1", "small"),
                        ("meta", "small"), ("full", "full"), ("2", "full")]:
        pack.reset()
        if value is None:
            monkeypatch.delenv("TERRACE_TA2A_PACK", raising=False)
        else:
            monkeypatch.setenv("TERRACE_TA2A_PACK", value)
        assert pack.pack_mode() == want and pack.pack_enabled() == (want != "off")
    pack.reset()
    monkeypatch.setenv("TERRACE_TA2A_PACK", "everything")
    with pytest.raises(ValueError):
        pack.pack_mode()
    pack.reset()
    monkeypatch.delenv("TERRACE_TA2A_PACK")


# ---- executable specs ---------------------------------------------------------------------------
K1_GEOMS = [(16, 2, 2, 8, 64), (64, 1, 2, 8, 32), (33, 3, 2, 4, 48), (128, 4, 4, 8, 16),
            (7, 2, 8, 4, 96), (1, 1, 1, 1, 24), (256, 2, 2, 16, 8), (40, 5, 3, 4, 40),
            (48, 7, 9, 7, 8)]


def _verbatim_chain(rx, rslot, rgate, quota, epr, rpn):
    """The arrival chain written the long way: expand pairs, stable sort by owner."""
    R = rslot.shape[0]
    r_idx = torch.arange(R).repeat_interleave(quota)
    slot = rslot.reshape(-1)
    owner = slot // epr
    order = torch.sort(owner, stable=True).indices
    return (rx[r_idx[order]], rgate.reshape(-1)[order], r_idx[order], slot[order],
            torch.bincount(owner, minlength=rpn))


@pytest.mark.parametrize("geom", K1_GEOMS)
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
def test_k1_ref_equals_verbatim_chain(geom, dt):
    R, q, epr, rpn, H = geom
    g = torch.Generator().manual_seed(R + q)
    rslot = torch.stack([torch.randperm(epr * rpn, generator=g)[:q].sort().values
                         for _ in range(R)])
    rx = torch.randn(R, H, generator=g).to(dt)
    rgate = torch.rand(R, q, generator=g).to(dt)
    for a, b in zip(k1_arrival_ref(rx, rslot, rgate, q, epr, rpn), _verbatim_chain(rx, rslot, rgate, q, epr, rpn)):
        assert torch.equal(a, b)


def test_k1_degenerate_and_backward():
    rx = torch.zeros(0, 8)
    out = k1_arrival_ref(rx, torch.zeros(0, 2, dtype=torch.long), torch.zeros(0, 2), 2, 2, 4)
    assert out[0].shape == (0, 8) and out[4].tolist() == [0, 0, 0, 0]
    with pytest.raises(AssertionError):
        k1_arrival_ref(torch.zeros(2, 4), torch.zeros(2, 3, dtype=torch.long), torch.zeros(2, 3),
                       2, 2, 2)
    g = torch.Generator().manual_seed(0)
    R, q, epr, rpn, H = 12, 2, 2, 4, 6
    rslot = torch.stack([torch.randperm(8, generator=g)[:q].sort().values for _ in range(R)])
    rx = torch.randn(R, H, generator=g, requires_grad=True)
    rgate = torch.rand(R, q, generator=g, requires_grad=True)
    for fn in (ops.k1_arrival, ops.k1_arrival_segment):
        send, gp, r_idx, slot_idx, i_send = fn(rx, rslot, rgate, q, epr, rpn, 1)
        w1, w2 = torch.randn_like(send), torch.randn_like(gp)
        grx, grg = torch.autograd.grad((send * w1).sum() + (gp * w2).sum(), (rx, rgate))
        ref = k1_arrival_ref(rx, rslot, rgate, q, epr, rpn)
        rrx, rrg = torch.autograd.grad((ref[0] * w1).sum() + (ref[1] * w2).sum(), (rx, rgate))
        torch.testing.assert_close(grx, rrx)
        torch.testing.assert_close(grg, rrg)
        assert not r_idx.requires_grad and int(i_send.sum()) == R * q
    send, gp, *_ = ops.k1_arrival_segment(rx, rslot, rgate, q, epr, rpn)
    send.sum().backward(retain_graph=False)          # two independent backward calls
    gp.sum().backward()
    with pytest.raises(ValueError):
        ops.k1_arrival(rx, rslot, rgate, q, epr, rpn, my_local=9)


K2_GEOMS = [(4, 2, 8, 8, 4, 2), (32, 8, 64, 48, 4, 2), (32, 8, 96, 32, 8, 4), (32, 8, 128, 32, 8, 2),
            (16, 8, 32, 5, 2, 2), (16, 4, 16, 12, 4, 1), (8, 4, 8, 1, 2, 2), (64, 8, 128, 33, 6, 3)]


@pytest.mark.parametrize("geom", K2_GEOMS)
@pytest.mark.parametrize("sort_rows", [True, False])
def test_k2_ref_equals_plan_gather_pack(geom, sort_rows):
    reset_plan_cache()
    world, rpn, E, T, k, M = geom
    idx = _quota_routing(T, E, world // rpn, k, M, T + k, sort_rows)
    g = torch.Generator().manual_seed(1)
    hidden = torch.randn(T, 12, generator=g)
    gates = torch.rand(T, k, generator=g)
    payload, mask, gate_rows, u_src, counts = k2_pack_ref(hidden, idx, gates, world, E, rpn, M)
    e_sorted, cols = idx.sort(dim=1)
    g_sorted = gates.gather(1, cols)
    pu, _, pc, inverse = plan_ta2a(e_sorted, world, E, rpn, groups_m=M)
    slots = (E // world) * rpn
    slot_tab, gate_tab, _ = pack_quota_wire(e_sorted, g_sorted, inverse, T * M, slots, k // M)
    assert torch.equal(u_src, pu) and torch.equal(counts, pc)
    assert torch.equal(payload, hidden[pu]) and torch.equal(mask, slot_tab)
    assert torch.equal(gate_rows, gate_tab)


def test_k2_validation_and_grad():
    h, idx, g = torch.randn(4, 6), torch.tensor([[0, 4], [1, 5], [2, 6], [3, 7]]), torch.rand(4, 2)
    with pytest.raises(RuntimeError):
        k2_pack_ref(h, idx, g.bfloat16(), 4, 8, 2, 2)
    with pytest.raises(ValueError):
        k2_pack_ref(h, idx, g, 4, 8, 3, 2)
    with pytest.raises(ValueError):
        k2_pack_ref(h, idx + 100, g, 4, 8, 2, 2)
    with pytest.raises(ValueError):
        k2_pack_ref(h, idx, g, 4, 8, 2, 2, max_slots=3)
    h.requires_grad_(True)
    g.requires_grad_(True)
    payload, _, gate_rows, u_src, _ = ops.k2_pack(h, idx, g, 4, 8, 2, 2)
    w1, w2 = torch.randn_like(payload), torch.randn_like(gate_rows)
    gh, gg = torch.autograd.grad((payload * w1).sum() + (gate_rows * w2).sum(), (h, g))
    ref = k2_pack_ref(h, idx, g, 4, 8, 2, 2)
    rh, rg = torch.autograd.grad((ref[0] * w1).sum() + (ref[2] * w2).sum(), (h, g))
    torch.testing.assert_close(gh, rh)
    torch.testing.assert_close(gg, rg)


def test_small_helpers():
    assert fixed_hist(torch.tensor([0, 2, 2, 5]), 6).tolist() == [1, 0, 2, 0, 0, 1]
    assert fixed_hist(torch.zeros(0, dtype=torch.long), 3).tolist() == [0, 0, 0]
    key = torch.tensor([2, 0, 2, 1, 0])
    assert stable_bucket_order(key, 3).tolist() == [1, 4, 3, 0, 2]


# ---- loader gate --------------------------------------------------------------------------------
def test_loader_tristate(monkeypatch, caplog, tmp_path):
    monkeypatch.setenv("TERRACE_OPS_LIB", str(tmp_path / "missing.so"))
    monkeypatch.setenv("TERRACE_CUSTOM_OPS", "0")
    ops.reset()
    assert not ops.custom_ops_enabled() and ops.status().requested == "0"
    monkeypatch.setenv("TERRACE_CUSTOM_OPS", "1")
    ops.reset()
    with caplog.at_level(logging.WARNING, logger="terrace.ops"):
        assert not ops.custom_ops_enabled()
        ops.custom_ops_enabled()                      # decided once: no second warning
    assert sum("falling back" in r.message for r in caplog.records) == 1
    monkeypatch.setenv("TERRACE_CUSTOM_OPS", "require")
    ops.reset()
    with pytest.raises(ops.OpsLoadError):
        ops.status()
    monkeypatch.setenv("TERRACE_CUSTOM_OPS", "sometimes")
    ops.reset()
    with pytest.raises(ValueError):
        ops.status()
    monkeypatch.delenv("TERRACE_CUSTOM_OPS")
    monkeypatch.delenv("TERRACE_OPS_LIB")
    ops.reset()
    if not torch.cuda.is_available():
        assert not ops.custom_ops_enabled()           # default without CUDA: off
    x = torch.randn(3, 4)
    y = ops.passthrough(x)
    assert torch.equal(x, y) and y.data_ptr() != x.data_ptr()
