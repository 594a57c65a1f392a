"""T-Route invariants, mode signatures, bias update, traffic matrix (CPU)."""
import pytest
import torch

from terracemoe_simulator_b200.bench import dispatch_traffic, uniformity_cv
from terracemoe_simulator_b200.routing import (ROUTING_MODES, Router, TRouteConfig, expert_load,
                                               t_route, update_bias_)


def _aff(T, E, seed=0):
    return torch.rand(T, E, generator=torch.Generator().manual_seed(seed))


@pytest.mark.parametrize("E,ng,k,m", [(64, 16, 4, 2), (64, 4, 6, 2), (32, 8, 8, 4), (16, 2, 4, 1),
                                       (256, 2, 8, 2)])
def test_full_mode_structural_guarantees(E, ng, k, m):
    cfg = TRouteConfig(E, ng, k, m)
    idx, gates, gidx = t_route(_aff(500, E), torch.zeros(E), cfg, "full")
    assert idx.shape == (500, k) and gidx.shape == (500, m) and idx.dtype == torch.int64
    groups = idx // cfg.group_size
    for t in range(0, 500, 37):
        assert len(set(idx[t].tolist())) == k
        per_group = torch.bincount(groups[t], minlength=ng)
        assert (per_group > 0).sum() == m
        assert set(per_group[per_group > 0].tolist()) == {k // m}
    torch.testing.assert_close(gates.sum(-1), torch.ones(500))
    assert (gates > 0).all()


def test_config_validation():
    with pytest.raises(ValueError):
        TRouteConfig(10, 4, 4, 2)
    with pytest.raises(ValueError):
        TRouteConfig(16, 4, 5, 2)
    with pytest.raises(ValueError):
        TRouteConfig(16, 8, 8, 2)         # quota 4 > group size 2
    cfg = TRouteConfig(16, 4, 4, 2)
    assert cfg.group_size == 4 and cfg.per_group_k == 2


def test_unknown_mode_raises():
    cfg = TRouteConfig(16, 4, 4, 2)
    for bad in ("Full", "quota", "", None):
        with pytest.raises(ValueError):
            t_route(_aff(4, 16), torch.zeros(16), cfg, bad)
    with pytest.raises(ValueError):
        Router(8, cfg)(torch.randn(3, 8), "nope")


def test_mode_signatures_and_distinctness():
    E, ng, k, m = 64, 16, 4, 2          # k divisible by n_groups? quota_only needs k % ng == 0
    cfg = TRouteConfig(64, 4, 4, 2)
    aff = _aff(2000, 64, 3)
    out = {mode: t_route(aff, torch.zeros(64), cfg, mode) for mode in ROUTING_MODES}
    span = {mode: (torch.stack([torch.bincount(r // cfg.group_size, minlength=4)
                                for r in out[mode][0]]) > 0).sum(1) for mode in ROUTING_MODES}
    assert (span["full"] == 2).all() and (span["group_limited"] <= 2).all()
    assert (span["quota_only"] == 4).all()
    assert span["global_topk"].float().mean() > 2.5
    assert out["quota_only"][2].shape == (2000, 4) and out["global_topk"][2].shape == (2000, 4)
    names = list(ROUTING_MODES)
    for i, a in enumerate(names):
        for b in names[i + 1:]:
            sa = out[a][0].sort(-1).values
            sb = out[b][0].sort(-1).values
            assert (sa != sb).any(-1).float().mean() > 0.25, (a, b)


def test_global_topk_matches_topk():
    cfg = TRouteConfig(32, 4, 4, 2)
    aff = _aff(100, 32, 5)
    bias = torch.randn(32) * 0.1
    idx, gates, _ = t_route(aff, bias, cfg, "global_topk")
    assert torch.equal(idx, (aff + bias).topk(4, -1).indices)
    raw = aff.gather(1, idx)
    torch.testing.assert_close(gates, raw / raw.sum(-1, keepdim=True))


def test_bias_update_lowers_load_cv():
    torch.manual_seed(0)
    cfg = TRouteConfig(32, 8, 4, 2)
    skew = torch.linspace(0.0, 0.6, 32)
    bias = torch.zeros(32)

    def cv():
        aff = torch.sigmoid(torch.randn(4096, 32) + skew)
        load = expert_load(t_route(aff, bias, cfg)[0], 32)
        return float(load.std() / load.mean()), load
    first, _ = cv()
    for _ in range(300):
        _, load = cv()
        update_bias_(bias, load, 5e-3)
    last, _ = cv()
    assert last < 0.6 * first


def test_update_bias_direction_and_inplace():
    bias = torch.zeros(4)
    out = update_bias_(bias, torch.tensor([10.0, 0.0, 5.0, 5.0]), 0.1)
    assert out is bias
    torch.testing.assert_close(bias, torch.tensor([-0.1, 0.1, 0.0, 0.0]))


def test_adversarial_affinity_group_cv():
    E, ng = 64, 16
    cfg = TRouteConfig(E, ng, 4, 2)
    aff = torch.rand(1000, E, generator=torch.Generator().manual_seed(1)) * 0.01
    aff[:, : 4 * cfg.group_size] += 1.0
    idx, _, gidx = t_route(aff, torch.zeros(E), cfg, "full")
    assert int(gidx.max()) < 4                    # every token lands in the boosted groups
    cfg_all = TRouteConfig(E, ng, 16, 16)
    idx2, _, _ = t_route(aff, torch.zeros(E), cfg_all, "quota_only")
    load = torch.bincount((idx2 // cfg_all.group_size).reshape(-1), minlength=ng).float()
    assert float(load.std()) == 0.0               # M == N_g: strictly balanced over groups


def test_traffic_matrix_dedup_invariant():
    cfg = TRouteConfig(64, 8, 6, 2)
    idx, _, gidx = t_route(_aff(512, 64, 7), torch.zeros(64), cfg)
    src = torch.arange(512) % 16
    mat = dispatch_traffic(gidx, src, cfg, cards_per_group=2)
    assert mat.shape == (8, 8) and int(mat.sum()) == 512 * 2     # one message per (token, group)
    assert uniformity_cv(mat) < 1.0


def test_router_module_and_softmax_option():
    cfg = TRouteConfig(16, 4, 4, 2)
    r = Router(32, cfg)
    assert r.weight.shape == (16, 32) and "bias" in dict(r.named_buffers())
    assert "bias" in r.state_dict()
    h = torch.randn(10, 32, requires_grad=True)
    idx, gates, gidx = r(h)
    gates.sum().backward()
    assert h.grad is not None and r.weight.grad is not None
    r2 = Router(32, cfg, score_func="softmax")
    _, g2, _ = r2(torch.randn(5, 32))
    torch.testing.assert_close(g2.sum(-1), torch.ones(5))
    with pytest.raises(ValueError):
        Router(32, cfg, score_func="relu")
