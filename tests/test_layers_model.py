"""Layers, decoder, aux loss, checkpoints (CPU)."""
import copy

import pytest
import torch
import torch.nn.functional as F

from terracemoe_simulator_b200.layer import (HierarchicalMoE, SwiGLU, TerracedMoE, apply_capacity,
                                             grouped_mm)
from terracemoe_simulator_b200.models import ModelArgs, TerraceLM, _balance_aux, rmsnorm
from terracemoe_simulator_b200.models.checkpoint import (load_checkpoint, merge_state_dicts,
                                                         save_checkpoint, shard_state_dict)
from terracemoe_simulator_b200.routing import ROUTING_MODES, TRouteConfig


def test_grouped_mm_matches_block_diagonal_with_empty_group():
    torch.manual_seed(0)
    counts = torch.tensor([3, 0, 5, 2])
    x = torch.randn(10, 6, requires_grad=True)
    w = torch.randn(4, 6, 7, requires_grad=True)
    y = grouped_mm(x, w, counts)
    ref = torch.cat([x[0:3] @ w[0], x[3:8] @ w[2], x[8:10] @ w[3]])
    torch.testing.assert_close(y, ref)
    gy = torch.randn_like(y)
    gx, gw = torch.autograd.grad(y, (x, w), gy)
    rx, rw = torch.autograd.grad(ref, (x, w), gy)
    torch.testing.assert_close(gx, rx)
    torch.testing.assert_close(gw, rw)
    assert torch.all(gw[1] == 0)


@pytest.mark.parametrize("mode", ROUTING_MODES)
def test_loop_and_grouped_backends_agree(mode):
    torch.manual_seed(1)
    cfg = TRouteConfig(16, 4, 4, 2)
    moe = TerracedMoE(24, 16, 32, cfg)
    moe.routing_mode = mode
    moe.eval()
    x = torch.randn(2, 9, 24)
    outs, grads = [], []
    for backend in ("loop", "grouped"):
        moe.expert_backend = backend
        moe.zero_grad()
        y, stats = moe(x)
        y.square().sum().backward()
        outs.append(y.detach())
        grads.append([p.grad.clone() for p in moe.parameters()])
        assert set(stats) >= {"expert_load", "group_idx", "gates", "expert_idx"}
    torch.testing.assert_close(outs[0], outs[1], rtol=1e-4, atol=1e-5)
    for a, b in zip(*grads):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)
    moe.expert_backend = "bogus"
    with pytest.raises(ValueError):
        moe(x)


def test_training_forward_updates_bias_eval_does_not():
    cfg = TRouteConfig(16, 4, 4, 2)
    moe = TerracedMoE(8, 8, 8, cfg)
    x = torch.randn(64, 8)
    moe.eval()
    moe(x)
    assert torch.all(moe.router.bias == 0)
    moe.train()
    moe(x)
    assert moe.router.bias.abs().sum() > 0


def test_capacity_factor_drops_in_canonical_order():
    idx = torch.tensor([[0, 1], [0, 2], [0, 3], [0, 1]])
    gates = torch.full((4, 2), 0.5)
    kept, keep, cap = apply_capacity(idx, gates, 4, 1.0)     # cap = ceil(8/4) = 2
    assert cap == 2
    assert keep[:, 0].tolist() == [True, True, False, False]  # expert 0: first two tokens only
    assert keep[:, 1].all()
    assert torch.equal(kept, gates * keep)
    _, keep2, _ = apply_capacity(idx, gates, 4, 1.0, prior_counts=torch.tensor([1, 0, 0, 0]))
    assert keep2[:, 0].tolist() == [True, False, False, False]
    g3, k3, c3 = apply_capacity(idx, gates, 4, None)
    assert c3 is None and k3.all() and g3 is gates
    moe = TerracedMoE(8, 8, 8, TRouteConfig(8, 2, 2, 1), capacity_factor=0.5)
    moe.eval()
    y, stats = moe(torch.randn(32, 8))
    assert "dropped" in stats and int(stats["dropped"]) > 0


def test_hierarchical_moe_runs_and_reports_hard_tokens():
    cfg = TRouteConfig(8, 2, 2, 1)
    h = HierarchicalMoE(16, 8, 32, 0.25, cfg)
    h.expert_backend = "grouped"
    y, stats = h(torch.randn(40, 16))
    assert y.shape == (40, 16) and stats["n_hard"] == 10
    # tier 1 has no shared expert, yet it keeps the two (zero-element) keys the reference's
    # HierarchicalMoE carries, so state dicts interchange with strict loading
    sd = h.state_dict()
    assert "tier0.shared.w13.weight" in sd
    assert sd["tier1.shared.w13.weight"].numel() == 0 and sd["tier1.shared.w2.weight"].numel() == 0
    assert tuple(sd["tier1.shared.w2.weight"].shape) == (16, 0)
    # n_shared = 0 on tier 0 as well: the layer runs and the shared branch contributes zero
    h0 = HierarchicalMoE(16, 8, 32, 0.25, cfg, n_shared=0)
    assert h0(torch.randn(8, 16))[0].shape == (8, 16)


def test_hierarchical_state_dict_round_trips_with_the_reference_model():
    """Strict loading in both directions against the reference's own TerraceLM (arch "hier")."""
    import importlib.util
    import os
    import sys
    ref_root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                            "baseline", "_ref")
    if not os.path.isfile(os.path.join(ref_root, "terrace", "model.py")):
        pytest.skip("no copy of the reference package beside the repository")
    saved = {k: v for k, v in sys.modules.items() if k == "terrace" or k.startswith("terrace.")}
    for k in saved:
        del sys.modules[k]
    sys.path.insert(0, ref_root)
    try:
        ref_model = importlib.import_module("terrace.model")
        kw = dict(vocab=64, dim=32, n_layers=2, n_heads=2, seq_len=16, n_experts=8, n_groups=2,
                  top_k=2, top_groups=1, arch="hier", d0=16, d1=32, dense_first=1)
        torch.manual_seed(0)
        theirs = ref_model.TerraceLM(ref_model.ModelArgs(**kw))
        ours = TerraceLM(ModelArgs(**kw))
        assert set(theirs.state_dict()) == set(ours.state_dict())
        ours.load_state_dict(theirs.state_dict(), strict=True)
        theirs.load_state_dict(ours.state_dict(), strict=True)
        ids = torch.randint(0, 64, (2, 16))
        theirs.eval(), ours.eval()
        torch.testing.assert_close(ours(ids)[0], theirs(ids)[0], rtol=1e-5, atol=1e-5)
    finally:
        sys.path.remove(ref_root)
        for k in [k for k in sys.modules if k == "terrace" or k.startswith("terrace.")]:
            del sys.modules[k]
        sys.modules.update(saved)


def test_rmsnorm_and_swiglu_formulas():
    x, w = torch.randn(3, 5, 8), torch.rand(8)
    torch.testing.assert_close(rmsnorm(x, w), x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w)
    s = SwiGLU(8, 12)
    a, b = s.w13(x).chunk(2, -1)
    torch.testing.assert_close(s(x), s.w2(F.silu(a) * b))


def _tiny_args(**kw):
    base = dict(vocab=64, dim=32, n_layers=4, n_heads=4, seq_len=16, n_experts=8, n_groups=4,
                top_k=4, top_groups=2, d_expert=16, d_shared=16, expert_backend="grouped")
    base.update(kw)
    return ModelArgs(**base)


def test_model_layer_layout_and_state_dict_keys():
    m = TerraceLM(_tiny_args())
    assert [b.is_moe for b in m.blocks] == [False, True, True, False]
    keys = set(m.state_dict())
    for k in ("tok.weight", "nf", "head.weight", "blocks.0.ffn.w13.weight", "blocks.0.ffn.w2.weight",
              "blocks.1.ffn.w13", "blocks.1.ffn.w2", "blocks.1.ffn.router.weight",
              "blocks.1.ffn.router.bias", "blocks.1.ffn.shared.w13.weight",
              "blocks.1.ffn.shared.w2.weight", "blocks.1.attn.wqkv.weight", "blocks.1.attn.wo.weight",
              "blocks.1.n1", "blocks.1.n2"):
        assert k in keys, k
    assert not any("cos" in k or "sin" in k or k.endswith("qn") for k in keys)
    every = TerraceLM(_tiny_args(moe_every_layer=True))
    assert all(b.is_moe for b in every.blocks)
    logits, info = m(torch.randint(0, 64, (2, 16)))
    assert logits.shape == (2, 16, 64) and info == {}
    with pytest.raises(ValueError):
        m(torch.randint(0, 64, (1, 17)))
    assert m.n_params() == sum(p.numel() for p in m.parameters())


def test_balance_aux_properties():
    a = _tiny_args()
    E = a.n_experts
    idx = torch.randint(0, E, (200, 4))
    gates = torch.rand(200, 4, requires_grad=True)
    load = torch.bincount(idx.reshape(-1), minlength=E).float()
    aux = _balance_aux([load], [gates], [idx], a)
    aux.backward()
    assert gates.grad is not None and gates.grad.abs().sum() > 0
    skew_idx = torch.zeros(200, 4, dtype=torch.long)
    skew_load = torch.bincount(skew_idx.reshape(-1), minlength=E).float()
    g = torch.full((200, 4), 0.25)
    assert _balance_aux([skew_load], [g], [skew_idx], a) > _balance_aux([load], [g], [idx], a)
    two = _balance_aux([load, load], [g, g], [idx, idx], a)
    torch.testing.assert_close(two, _balance_aux([load], [g], [idx], a))
    m = TerraceLM(a)
    x = torch.randint(0, 64, (2, 16))
    loss, info = m(x, x)
    assert set(info) == {"lm_loss", "aux", "loads", "routes"} and info["routes"] == []
    m.collect_routes = True
    assert len(m(x, x)[1]["routes"]) == 2


def _train(model, opt, gen, steps):
    for _ in range(steps):
        x = torch.randint(0, 64, (2, 16), generator=gen)
        loss, _ = model(x, x)
        opt.zero_grad()
        loss.backward()
        opt.step()
    return loss.item()


def test_checkpoint_resume_equals_uninterrupted(tmp_path):
    torch.manual_seed(0)
    base = TerraceLM(_tiny_args())
    m1, m2 = copy.deepcopy(base), copy.deepcopy(base)
    o1 = torch.optim.AdamW(m1.parameters(), lr=1e-3)
    g1 = torch.Generator().manual_seed(5)
    _train(m1, o1, g1, 10)
    o2 = torch.optim.AdamW(m2.parameters(), lr=1e-3)
    g2 = torch.Generator().manual_seed(5)
    _train(m2, o2, g2, 6)
    path = tmp_path / "ck.pt"
    save_checkpoint(path, m2, o2, g2)
    blob = torch.load(path, weights_only=False)
    assert set(blob) == {"model", "opt", "gen"}
    m3 = TerraceLM(_tiny_args())
    o3 = torch.optim.AdamW(m3.parameters(), lr=1e-3)
    g3 = torch.Generator()
    load_checkpoint(path, m3, o3, g3)
    _train(m3, o3, g3, 4)
    for (k, a), b in zip(m1.state_dict().items(), m3.state_dict().values()):
        torch.testing.assert_close(a, b, rtol=0, atol=1e-5, msg=k)


def test_expert_shard_round_trip():
    m = TerraceLM(_tiny_args())
    full = m.state_dict()
    shards = [shard_state_dict(full, r, 4) for r in range(4)]
    assert shards[1]["blocks.1.ffn.w13"].shape[0] == 2
    assert torch.equal(shards[2]["blocks.1.ffn.w2"], full["blocks.1.ffn.w2"][4:6])
    merged = merge_state_dicts(shards)
    for k in full:
        assert torch.equal(merged[k], full[k]), k
    shards[1]["nf"] = shards[1]["nf"] + 1
    with pytest.raises(ValueError):
        merge_state_dicts(shards)
    with pytest.raises(ValueError):
        shard_state_dict(full, 0, 3)


@pytest.mark.parametrize("chunk", [5, 16, 64])
def test_chunked_lm_loss_equals_the_unchunked_loss_and_gradients(chunk):
    import torch.nn.functional as F
    from terracemoe_simulator_b200.models.decoder import chunked_lm_loss
    torch.manual_seed(0)
    n, d, v = 37, 24, 50                                   # 37 tokens: the last chunk is ragged
    h0, w0 = torch.randn(n, d), torch.randn(v, d) * d ** -0.5
    tgt = torch.randint(0, v, (n,))
    h1, w1 = h0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
    ref = F.cross_entropy(F.linear(h1, w1).float(), tgt)
    (3.0 * ref).backward()
    h2, w2 = h0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
    got = chunked_lm_loss(h2, w2, tgt, chunk)
    (3.0 * got).backward()
    torch.testing.assert_close(got, ref, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(h2.grad, h1.grad, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(w2.grad, w1.grad, rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        chunked_lm_loss(h2, w2, tgt, 0)


def test_model_with_chunked_loss_trains_like_the_unchunked_model():
    from terracemoe_simulator_b200.models import ModelArgs, TerraceLM
    kw = dict(vocab=64, dim=32, n_layers=3, n_heads=2, seq_len=16, n_experts=8, n_groups=4, top_k=2,
              top_groups=1, d_expert=16, d_shared=16, expert_backend="grouped")
    torch.manual_seed(1)
    a = TerraceLM(ModelArgs(**kw))
    torch.manual_seed(1)
    b = TerraceLM(ModelArgs(ce_chunk=10, **kw))
    idx = torch.randint(0, 64, (3, 17))
    la, _ = a(idx[:, :-1], idx[:, 1:])
    lb, _ = b(idx[:, :-1], idx[:, 1:])
    la.backward()
    lb.backward()
    torch.testing.assert_close(la, lb, rtol=1e-6, atol=1e-6)
    for (n1, p1), (_, p2) in zip(a.named_parameters(), b.named_parameters()):
        if p1.grad is not None:
            torch.testing.assert_close(p1.grad, p2.grad, rtol=2e-5, atol=1e-6, msg=n1)
    with torch.no_grad():                                   # evaluation takes the plain path
        assert torch.isfinite(b(idx[:, :-1], idx[:, 1:])[0])
