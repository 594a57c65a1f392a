"""GPU numerics: every CUDA kernel against a plain PyTorch fp32 reference of the same op."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _close(a, b, rtol=2e-2, atol=None):
    a, b = a.float(), b.float()
    scale = b.abs().max().item() + 1e-6
    atol = atol if atol is not None else 1e-2 * scale
    torch.testing.assert_close(a, b, rtol=rtol, atol=atol)


def test_passthrough_bitwise(native_ops):
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        for shape in ((7,), (33, 65), (4, 128, 96)):
            x = torch.randn(*shape, device=DEV).to(dt)
            y = native_ops.passthrough(x)
            assert y.data_ptr() != x.data_ptr() and torch.equal(x, y)
    assert native_ops.OP_CALLS.get("passthrough", 0) > 0


# widths that reach each backward kernel: generic (96), 16-byte loads (512), and the column-split
# kernel with 4..8 warps and 1..4 column groups per lane; row counts that leave ragged row batches
RMSNORM_SHAPES = [((37, 5), 512), ((37, 5), 96), ((3001,), 1024), ((3001,), 4096), ((1201,), 1536),
                  ((700,), 7168), ((1000,), 6144), ((611,), 2048), ((300,), 8192), ((500,), 5120)]


@pytest.mark.parametrize("shape", RMSNORM_SHAPES)
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_rmsnorm_fwd_bwd(native_ops, dt, shape):
    torch.manual_seed(0)
    lead, dim = shape
    x = torch.randn(*lead, dim, device=DEV).to(dt).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(dim, device=DEV)).to(dt).requires_grad_(True)
    y = native_ops.rmsnorm(x, w, 1e-5)
    gy = torch.randn_like(y)
    y.backward(gy)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    yr.backward(gy.float())
    tol = 1e-5 if dt == torch.float32 else 2e-2
    torch.testing.assert_close(y.float(), yr, rtol=tol, atol=tol)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=tol, atol=tol)
    # the weight gradient sums over all rows: its rounding grows with the row count
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=tol, atol=tol * 10 * max(1.0, (x.numel() / dim / 185) ** 0.5))


K1_GEOMS = [(16, 2, 2, 8, 64), (64, 1, 2, 8, 32), (33, 3, 2, 4, 48), (128, 4, 4, 8, 16),
            (7, 2, 8, 4, 96), (1, 1, 1, 1, 24), (256, 2, 2, 16, 8), (40, 5, 3, 4, 40),
            (48, 7, 9, 7, 8), (2000, 4, 32, 4, 256)]


@pytest.mark.parametrize("geom", K1_GEOMS)
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
def test_k1_arrival_bitwise(native_ops, geom, dt):
    R, q, epr, rpn, H = geom
    g = torch.Generator().manual_seed(R * 31 + q)
    slots = epr * rpn
    rslot = torch.stack([torch.randperm(slots, generator=g)[:q].sort().values for _ in range(R)])
    rx = torch.randn(R, H, generator=g).to(dt)
    rgate = torch.rand(R, q, generator=g).to(dt)
    ref = native_ops.k1_arrival_ref(rx, rslot, rgate, q, epr, rpn, 0)
    got = torch.ops.terrace.k1_arrival(rx.to(DEV), rslot.to(DEV), rgate.to(DEV), q, epr, rpn, 0)
    for a, b in zip(got, ref):
        assert torch.equal(a.cpu(), b)


def test_k1_arrival_empty(native_ops):
    rx = torch.zeros(0, 16, device=DEV)
    out = torch.ops.terrace.k1_arrival(rx, torch.zeros(0, 2, dtype=torch.long, device=DEV),
                                       torch.zeros(0, 2, device=DEV), 2, 2, 4, 0)
    assert out[0].shape == (0, 16) and out[4].tolist() == [0, 0, 0, 0]


K2_GEOMS = [(4, 2, 8, 8, 4, 2), (32, 8, 64, 48, 4, 2), (32, 8, 96, 32, 8, 4), (32, 8, 128, 32, 8, 2),
            (16, 8, 32, 5, 2, 2), (16, 4, 16, 12, 4, 1), (8, 4, 8, 1, 2, 2), (64, 8, 128, 33, 6, 3),
            (8, 4, 256, 777, 8, 2)]


def _quota_routing(T, E, n_nodes, k, M, g, sort_rows):
    per = E // n_nodes
    q = k // M
    rows = []
    for _ in range(T):
        groups = torch.randperm(n_nodes, generator=g)[:M]
        picks = torch.cat([grp * per + torch.randperm(per, generator=g)[:q] for grp in groups])
        picks = picks[torch.randperm(k, generator=g)]
        rows.append(picks.sort().values if sort_rows else picks)
    return torch.stack(rows)


@pytest.mark.parametrize("geom", K2_GEOMS)
@pytest.mark.parametrize("sort_rows", [True, False])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_k2_pack_bitwise(native_ops, geom, sort_rows, dt):
    world, rpn, E, T, k, M = geom
    g = torch.Generator().manual_seed(T * 7 + k)
    idx = _quota_routing(T, E, world // rpn, k, M, g, sort_rows)
    hidden = torch.randn(T, 40, generator=g).to(dt)
    gates = torch.rand(T, k, generator=g).to(dt)
    ref = native_ops.k2_pack_ref(hidden, idx, gates, world, E, rpn, M)
    got = torch.ops.terrace.k2_pack(hidden.to(DEV), idx.to(DEV), gates.to(DEV), world, E, rpn, M)
    for a, b in zip(got, ref):
        assert torch.equal(a.cpu(), b)


@pytest.mark.parametrize("T,E,k,align", [(300, 16, 4, 1), (1000, 16, 4, 64), (5000, 64, 6, 64),
                                         (33, 8, 2, 1), (4096, 256, 8, 64)])
def test_moe_plan_is_the_stable_counting_sort(native_ops, T, E, k, align):
    """Rows of an expert are ordered by token (the canonical order the capacity rule relies on):
    position = segment start + earlier tokens that picked the expert."""
    g = torch.Generator().manual_seed(T + E)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    gates = torch.rand(T, k, generator=g)
    es, gs, cols, pos, seg_start, seg_count = torch.ops.terrace.moe_plan(idx.to(DEV), gates.to(DEV),
                                                                         E, align)
    order = torch.argsort(idx, dim=1, stable=True)
    want_es = idx.gather(1, order)
    counts = torch.bincount(idx.reshape(-1), minlength=E)
    padded = (counts + align - 1) // align * align
    start = torch.cumsum(padded, 0) - padded
    onehot = torch.zeros(T, E, dtype=torch.long).scatter_add_(1, idx, torch.ones_like(idx))
    earlier = torch.cumsum(onehot, 0) - onehot
    want_pos = start[want_es] + earlier.gather(1, want_es)
    assert torch.equal(es.cpu().long(), want_es) and torch.equal(cols.cpu().long(), order)
    assert torch.equal(gs.cpu(), gates.gather(1, order))
    assert torch.equal(seg_count.cpu().long(), counts) and torch.equal(seg_start.cpu().long(), start)
    assert torch.equal(pos.cpu().long(), want_pos)


def test_moe_plan_with_a_repeated_expert_still_tiles(native_ops):
    """Not a top-k routing (a token names an expert twice): every pick still gets its own row
    inside the expert's segment."""
    g = torch.Generator().manual_seed(3)
    T, E, k = 700, 8, 4
    idx = torch.randint(0, E, (T, k), generator=g)
    es, _, _, pos, seg_start, seg_count = torch.ops.terrace.moe_plan(idx.to(DEV), None, E, 1)
    pos, es = pos.cpu().long().reshape(-1), es.cpu().long().reshape(-1)
    assert torch.equal(torch.sort(pos).values, torch.arange(T * k))
    lo = seg_start.cpu().long()[es]
    assert bool(((pos >= lo) & (pos < lo + seg_count.cpu().long()[es])).all())


def test_route_select_matches_t_route(native_ops):
    from terracemoe_simulator_b200.routing import TRouteConfig, t_route
    torch.manual_seed(1)
    for (E, ng, k, M, T) in [(64, 4, 6, 2, 1000), (64, 16, 4, 2, 513), (256, 2, 8, 2, 300),
                             (16, 2, 4, 1, 77)]:
        cfg = TRouteConfig(E, ng, k, M)
        logits = torch.randn(T, E, device=DEV)
        bias = 0.01 * torch.randn(E, device=DEV)
        idx, gates, gidx, load = native_ops.route_from_logits(logits, bias, cfg)
        ridx, rgates, rgidx = t_route(torch.sigmoid(logits), bias, cfg, "full")
        same = (idx == ridx).all(dim=1)
        assert same.float().mean() > 0.995
        torch.testing.assert_close(gates[same], rgates[same], rtol=1e-4, atol=1e-5)
        assert torch.equal(gidx[same], rgidx[same])
        assert load.sum().item() == T * k


def test_route_select_backward(native_ops):
    from terracemoe_simulator_b200.routing import TRouteConfig, t_route
    torch.manual_seed(2)
    cfg = TRouteConfig(64, 4, 6, 2)
    logits = torch.randn(200, 64, device=DEV, requires_grad=True)
    bias = torch.zeros(64, device=DEV)
    idx, gates, _, _ = native_ops.route_from_logits(logits, bias, cfg)
    w = torch.randn_like(gates)
    (gates * w).sum().backward()
    l2 = logits.detach().clone().requires_grad_(True)
    ridx, rgates, _ = t_route(torch.sigmoid(l2), bias, cfg, "full")
    assert torch.equal(idx, ridx)
    (rgates * w).sum().backward()
    torch.testing.assert_close(logits.grad, l2.grad, rtol=1e-3, atol=1e-6)


def test_rope_split_matches_the_eager_chain(native_ops):
    """Head split + RoPE in one kernel against the reference formula (fp32, rounded once), forward
    and backward."""
    from terracemoe_simulator_b200.models.decoder import _rope
    torch.manual_seed(6)
    B, T, nh, hd = 2, 200, 4, 64
    D = nh * hd
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd))
    angle = torch.outer(torch.arange(256).float(), inv_freq).to(DEV)
    cos, sin = angle.cos()[None, None], angle.sin()[None, None]
    qkv = torch.randn(B, T, 3 * D, device=DEV).bfloat16().requires_grad_(True)
    q, k, v = native_ops.rope_split(qkv, cos[..., :T, :], sin[..., :T, :], nh)
    gq, gk, gv = (torch.randn_like(q) for _ in range(3))
    torch.autograd.backward((q, k, v), (gq, gk, gv))
    ref = qkv.detach().clone().requires_grad_(True)
    rq, rk, rv = (t.view(B, T, nh, hd).transpose(1, 2) for t in ref.chunk(3, dim=-1))
    rq = _rope(rq, cos[..., :T, :], sin[..., :T, :]).to(rv.dtype)
    rk = _rope(rk, cos[..., :T, :], sin[..., :T, :]).to(rv.dtype)
    assert torch.equal(q, rq) and torch.equal(k, rk) and torch.equal(v, rv)
    torch.autograd.backward((rq, rk, rv), (gq, gk, gv))
    torch.testing.assert_close(qkv.grad.float(), ref.grad.float(), rtol=2e-2, atol=2e-2)
    assert q.is_contiguous() and tuple(q.shape) == (B, nh, T, hd)


def test_route_fused_matches_fp32_oracle(native_ops):
    """Router GEMM + selection in one launch against x @ W^T in fp32 followed by ``t_route``."""
    from terracemoe_simulator_b200.ops import native
    from terracemoe_simulator_b200.routing import TRouteConfig, expert_load, t_route
    torch.manual_seed(3)
    for (E, ng, k, M, T, H) in [(64, 4, 6, 2, 1000, 512), (128, 8, 8, 4, 300, 256),
                                (16, 2, 4, 1, 77, 64), (48, 3, 3, 3, 130, 320),
                                (64, 4, 6, 2, 4096, 4096)]:
        cfg = TRouteConfig(E, ng, k, M)
        x = torch.randn(T, H, device=DEV).bfloat16()
        w = (torch.randn(E, H, device=DEV) * H ** -0.5).bfloat16()
        bias = 0.01 * torch.randn(E, device=DEV)
        before = native.LIVE["route_fused"]
        idx, gates, gidx, load = native_ops.route_hidden(x, w, bias, cfg)
        assert native.LIVE["route_fused"] == before + 1
        logits = x.float() @ w.float().t()
        ridx, rgates, rgidx = t_route(torch.sigmoid(logits), bias, cfg, "full")
        same = (idx == ridx).all(dim=1)
        assert same.float().mean() > 0.99, (E, same.float().mean().item())
        torch.testing.assert_close(gates[same], rgates[same], rtol=2e-4, atol=1e-5)
        assert torch.equal(gidx[same], rgidx[same])
        assert torch.equal(load, expert_load(idx, E))
        torch.testing.assert_close(gates.sum(dim=1), torch.ones(T, device=DEV), rtol=1e-5, atol=1e-5)
    assert native.take_status(0) == 0


def test_route_fused_backward(native_ops):
    from terracemoe_simulator_b200.routing import TRouteConfig
    torch.manual_seed(4)
    E, H, T = 64, 512, 600
    cfg = TRouteConfig(E, 4, 6, 2)
    x = torch.randn(T, H, device=DEV).bfloat16().requires_grad_(True)
    w = (torch.randn(E, H, device=DEV) * H ** -0.5).bfloat16().requires_grad_(True)
    bias = torch.zeros(E, device=DEV)
    idx, gates, _, _ = native_ops.route_hidden(x, w, bias, cfg)
    coef = torch.randn_like(gates)
    (gates * coef).sum().backward()
    # oracle: the same picks, gates recomputed in fp32 with autograd
    xf = x.detach().float().requires_grad_(True)
    wf = w.detach().float().requires_grad_(True)
    aff = torch.sigmoid(xf @ wf.t()).gather(1, idx)
    rg = aff / aff.sum(dim=1, keepdim=True)
    torch.testing.assert_close(gates, rg.detach(), rtol=2e-4, atol=1e-5)
    (rg * coef).sum().backward()
    for got, want in ((x.grad, xf.grad), (w.grad, wf.grad)):
        scale = want.abs().max().item()
        torch.testing.assert_close(got.float(), want, rtol=3e-2, atol=3e-2 * scale)


def _segs(counts):
    c = torch.tensor(counts, dtype=torch.int32, device=DEV)
    return (torch.cumsum(c, 0, dtype=torch.int32) - c), c


GEMM_CASES = [
    # counts, K, N
    ([128], 64, 256),
    ([300, 0, 77, 129], 256, 512),
    ([5, 1000, 3], 192, 264),
    ([257] * 8, 4096, 1408),
]


@pytest.mark.parametrize("counts,K,N", GEMM_CASES)
def test_grouped_gemm_fwd(native_ops, counts, K, N):
    torch.manual_seed(0)
    G, rows = len(counts), sum(counts)
    A = torch.randn(rows, K, device=DEV, dtype=torch.bfloat16)
    B = (torch.randn(G, K, N, device=DEV) * K ** -0.5).bfloat16()
    s, c = _segs(counts)
    C, _ = torch.ops.terrace.grouped_gemm(A, B, s, c, 0, 0, False, 0)
    ref = torch.empty(rows, N, device=DEV)
    off = 0
    for g, n in enumerate(counts):
        ref[off:off + n] = A[off:off + n].float() @ B[g].float()
        off += n
    _close(C, ref)
    assert native_ops.take_status() == 0


@pytest.mark.parametrize("counts,K,N", GEMM_CASES)
def test_grouped_gemm_dgrad(native_ops, counts, K, N):
    torch.manual_seed(0)
    G, rows = len(counts), sum(counts)
    A = torch.randn(rows, K, device=DEV, dtype=torch.bfloat16)
    B = (torch.randn(G, N, K, device=DEV) * K ** -0.5).bfloat16()
    s, c = _segs(counts)
    C, _ = torch.ops.terrace.grouped_gemm(A, B, s, c, 1, 0, False, 0)
    ref = torch.empty(rows, N, device=DEV)
    off = 0
    for g, n in enumerate(counts):
        ref[off:off + n] = A[off:off + n].float() @ B[g].float().t()
        off += n
    _close(C, ref)
    assert native_ops.take_status() == 0


@pytest.mark.parametrize("counts,M,N", [([64], 128, 256), ([300, 0, 77, 129], 256, 512),
                                          ([5, 1000, 3], 192, 264), ([700] * 4, 1024, 1408)])
def test_grouped_wgrad(native_ops, counts, M, N):
    torch.manual_seed(0)
    G, rows = len(counts), sum(counts)
    X = torch.randn(rows, M, device=DEV, dtype=torch.bfloat16)
    dY = torch.randn(rows, N, device=DEV, dtype=torch.bfloat16)
    s, c = _segs(counts)
    dW = torch.ops.terrace.grouped_wgrad(X, dY, s, c, 0)
    ref = torch.zeros(G, M, N, device=DEV)
    off = 0
    for g, n in enumerate(counts):
        ref[g] = X[off:off + n].float().t() @ dY[off:off + n].float()
        off += n
    _close(dW, ref)
    assert native_ops.take_status() == 0


@pytest.mark.parametrize("mode", [0, 1])
def test_grouped_gemm_swiglu_epilogue(native_ops, mode):
    torch.manual_seed(0)
    counts, K, d = [200, 31, 0, 400], 512, 384
    G, rows = len(counts), sum(counts)
    A = torch.randn(rows, K, device=DEV, dtype=torch.bfloat16)
    W = (torch.randn(G, K, 2 * d, device=DEV) * K ** -0.5).bfloat16()
    B = W if mode == 0 else W.transpose(1, 2).contiguous()
    s, c = _segs(counts)
    act, pre = torch.ops.terrace.grouped_gemm(A, B, s, c, mode, 1, True, 0)
    ref = torch.empty(rows, 2 * d, device=DEV)
    off = 0
    for g, n in enumerate(counts):
        ref[off:off + n] = A[off:off + n].float() @ W[g].float()
        off += n
    _close(pre, ref)
    gate, up = pre.float().chunk(2, dim=-1)
    _close(act, F.silu(gate) * up, rtol=1e-2)
    assert native_ops.take_status() == 0


def test_linear_and_ffn_autograd(native_ops):
    torch.manual_seed(0)
    x = torch.randn(3, 100, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(384, 256, device=DEV) * 256 ** -0.5).bfloat16().requires_grad_(True)
    y = native_ops.linear(x, w)
    gy = torch.randn_like(y)
    y.backward(gy)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = xr @ wr.t()
    yr.backward(gy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)
    _close(w.grad, wr.grad)

    w13 = (torch.randn(2 * 512, 256, device=DEV) * 256 ** -0.5).bfloat16().requires_grad_(True)
    w2 = (torch.randn(256, 512, device=DEV) * 512 ** -0.5).bfloat16().requires_grad_(True)
    x2 = x.detach().clone().requires_grad_(True)
    y = native_ops.swiglu_ffn(x2, w13, w2)
    y.backward(gy[..., :256].contiguous())
    xr = x.detach().float().requires_grad_(True)
    w13r, w2r = w13.detach().float().requires_grad_(True), w2.detach().float().requires_grad_(True)
    a, b = (xr @ w13r.t()).chunk(2, -1)
    yr = (F.silu(a) * b) @ w2r.t()
    yr.backward(gy[..., :256].float())
    _close(y, yr, rtol=5e-2)
    _close(x2.grad, xr.grad, rtol=5e-2)
    _close(w13.grad, w13r.grad, rtol=5e-2)
    _close(w2.grad, w2r.grad, rtol=5e-2)
    assert native_ops.take_status() == 0


def test_moe_experts_local_fwd_bwd(native_ops):
    from terracemoe_simulator_b200.routing import TRouteConfig, t_route
    torch.manual_seed(0)
    T, H, d, E, ng, k, M = 777, 256, 128, 16, 4, 4, 2
    cfg = TRouteConfig(E, ng, k, M)
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w13 = (torch.randn(E, H, 2 * d, device=DEV) * H ** -0.5).bfloat16().requires_grad_(True)
    w2 = (torch.randn(E, d, H, device=DEV) * d ** -0.5).bfloat16().requires_grad_(True)
    aff = torch.sigmoid(torch.randn(T, E, device=DEV))
    idx, gates, _ = t_route(aff, torch.zeros(E, device=DEV), cfg)
    gates = gates.detach().requires_grad_(True)
    y = native_ops.moe_experts_local(x, idx, gates, w13, w2, cfg.group_size)
    gy = torch.randn_like(y)
    y.backward(gy)

    xr = x.detach().float().requires_grad_(True)
    w13r, w2r = w13.detach().float().requires_grad_(True), w2.detach().float().requires_grad_(True)
    gr = gates.detach().clone().requires_grad_(True)
    yr = torch.zeros(T, H, device=DEV)
    for e in range(E):
        tok, col = (idx == e).nonzero(as_tuple=True)
        a, b = (xr[tok] @ w13r[e]).chunk(2, -1)
        yr = yr.index_add(0, tok, gr[tok, col, None] * ((F.silu(a) * b) @ w2r[e]))
    yr.backward(gy.float())
    _close(y, yr, rtol=5e-2)
    _close(x.grad, xr.grad, rtol=5e-2)
    _close(gates.grad, gr.grad, rtol=5e-2)
    _close(w13.grad, w13r.grad, rtol=5e-2)
    _close(w2.grad, w2r.grad, rtol=5e-2)
    assert native_ops.take_status() == 0
    # determinism: same inputs, same bits
    y2 = native_ops.moe_experts_local(x, idx, gates, w13, w2, cfg.group_size)
    assert torch.equal(y, y2)


def test_padded_segments_gemm_and_wgrad(native_ops):
    """Segments aligned to 64 rows: fwd/dgrad write zero padding rows, wgrad relies on them."""
    torch.manual_seed(3)
    lib = torch.ops.terrace
    counts, K, N, A = [70, 0, 129, 64, 5], 256, 320, 64
    G = len(counts)
    c = torch.tensor(counts, dtype=torch.int32, device=DEV)
    padded = (c + A - 1) // A * A
    s = (torch.cumsum(padded, 0, dtype=torch.int32) - padded).to(torch.int32)
    rows = int(padded.sum())
    X = torch.full((rows, K), float("nan"), device=DEV, dtype=torch.bfloat16)   # poison padding
    W = (torch.randn(G, K, N, device=DEV) * K ** -0.5).bfloat16()
    for g, n in enumerate(counts):
        X[int(s[g]):int(s[g]) + n] = torch.randn(n, K, device=DEV).bfloat16()
    lib.zero_pad_rows(X, s, c, A)
    Y, _ = lib.grouped_gemm(X, W, s, c, 0, 0, False, 0, A)
    dY = torch.randn(rows, N, device=DEV, dtype=torch.bfloat16)
    lib.zero_pad_rows(dY, s, c, A)
    dW = lib.grouped_wgrad(X, dY, s, c, 0, A)
    for g, n in enumerate(counts):
        a, b = int(s[g]), int(s[g]) + n
        if n == 0:
            assert torch.all(dW[g] == 0)
            continue
        _close(Y[a:b], X[a:b].float() @ W[g].float())
        assert torch.all(Y[b:int(s[g]) + int(padded[g])] == 0)
        _close(dW[g], X[a:b].float().t() @ dY[a:b].float())
    assert torch.isfinite(dW.float()).all()
    assert native_ops.take_status() == 0


def test_gemm_cta_pair_variant_in_subprocess(native_ops):
    """The pair policy is read once per process, so the cta_group::2 variants of every GEMM test
    run in a child process with TERRACE_GEMM_PAIR=1 (the default policy only pairs long groups)."""
    import os
    import subprocess
    import sys
    if os.environ.get("TERRACE_GEMM_PAIR") == "1":
        pytest.skip("already inside the pair run")
    env = dict(os.environ, TERRACE_GEMM_PAIR="1")
    proc = subprocess.run([sys.executable, "-m", "pytest", os.path.abspath(__file__), "-q", "-x", "-k",
                           "grouped or swiglu or padded or linear or moe_experts or long_groups"],
                          env=env, capture_output=True, timeout=900)
    assert proc.returncode == 0, proc.stdout.decode()[-3000:] + proc.stderr.decode()[-2000:]


@pytest.mark.parametrize("mode,counts", [(1, [300, 0, 129, 64]), (0, [1000]), (1, [1100, 1300, 1024, 2048])])
def test_swiglu_backward_epilogue_equals_gemm_then_swiglu_bwd(native_ops, mode, counts):
    """d(act) GEMM with the SwiGLU backward in its epilogue against the same GEMM followed by the
    stand-alone kernel (which reads the bf16 d(act) back from memory), short and long groups."""
    lib = torch.ops.terrace
    torch.manual_seed(5)
    G, H, d, pad = len(counts), 256, 192, 64
    cnt = torch.tensor(counts, dtype=torch.int32, device=DEV)
    padded = (cnt + pad - 1) // pad * pad
    st = (torch.cumsum(padded, 0) - padded).to(torch.int32)
    rows = int(padded.sum())
    dout = torch.randn(rows, H, device=DEV, dtype=torch.bfloat16)
    w2 = (torch.randn(G, d, H, device=DEV) * d ** -0.5).bfloat16()
    B = w2 if mode == 1 else w2.transpose(1, 2).contiguous()         # mode 0 wants [G, K, N]
    h13 = torch.randn(rows, 2 * d, device=DEV, dtype=torch.bfloat16)
    dact, _ = lib.grouped_gemm(dout, B, st, cnt, mode, 0, False, 0, pad)
    want = lib.swiglu_bwd(h13, dact)
    got = torch.full_like(h13, float("nan"))
    lib.grouped_gemm_ex(dout, B, got, h13, st, cnt, mode, 3, None, 0, 0, 0, 0, pad)
    torch.cuda.synchronize()
    for s0, c0, p0 in zip(st.tolist(), counts, padded.tolist()):
        a, b = got[s0:s0 + c0].float(), want[s0:s0 + c0].float()
        if c0:
            torch.testing.assert_close(a, b, rtol=2e-2, atol=2e-2 * b.abs().max().item())
        assert bool((got[s0 + c0:s0 + p0] == 0).all())                 # padding rows: zeros
    assert native_ops.take_status(0) == 0


def test_long_groups_use_pairs_by_default(native_ops):
    """Groups of 1024+ rows take the 256-row pair tiles under the default policy."""
    torch.manual_seed(1)
    counts, K, N = [1100, 1300, 1024, 2048], 512, 640
    G, rows = len(counts), sum(counts)
    A = torch.randn(rows, K, device=DEV, dtype=torch.bfloat16)
    B = (torch.randn(G, K, N, device=DEV) * K ** -0.5).bfloat16()
    s, c = _segs(counts)
    C, _ = torch.ops.terrace.grouped_gemm(A, B, s, c, 0, 0, False, 0)
    Ct, _ = torch.ops.terrace.grouped_gemm(A, B.transpose(1, 2).contiguous(), s, c, 1, 0, False, 0)
    off = 0
    for g, n in enumerate(counts):
        ref = A[off:off + n].float() @ B[g].float()
        _close(C[off:off + n], ref)
        _close(Ct[off:off + n], ref)
        off += n
    assert native_ops.take_status() == 0


def test_device_prefetcher_on_gpu(native_ops):
    import itertools
    from terracemoe_simulator_b200.utils.prefetch import DevicePrefetcher
    host = [torch.full((1024, 1024), float(i)).pin_memory() for i in range(3)]
    feed = DevicePrefetcher(itertools.cycle(host), DEV)
    acc = torch.zeros(1024, 1024, device=DEV)
    for step in range(9):
        x = next(feed)
        assert x.is_cuda
        acc += x @ torch.eye(1024, device=DEV)          # compute that overlaps the next copy
        assert float(x[0, 0]) == float(step % 3)
    torch.cuda.synchronize()
    assert float(acc[0, 0]) == 3 * (0 + 1 + 2)
    assert feed.copied_bytes >= 9 * 4 * 1024 * 1024


def test_prefetcher_refill_after_an_event_and_side_stream_readback(native_ops):
    """A copy gated on a compute-stream event still delivers the batches in order, and a value
    read back on its own stream equals the one read on the compute stream."""
    import itertools
    from terracemoe_simulator_b200.utils.prefetch import DeferredScalar, DevicePrefetcher
    host = [torch.full((512, 512), float(i)).pin_memory() for i in range(3)]
    feed = DevicePrefetcher(itertools.cycle(host), DEV, depth=2)
    plain, side = DeferredScalar(DEV, lag=2), DeferredScalar(DEV, lag=2, side_stream=True)
    got_plain, got_side = [], []
    for step in range(8):
        x = feed.take()
        y = (x @ torch.eye(512, device=DEV)).sum() / (512 * 512)
        mark = torch.cuda.Event()
        mark.record()
        feed.refill(after=mark)
        got_plain.append(plain.push(y))
        got_side.append(side.push(y))
    want = [None, None] + [float(i % 3) for i in range(6)]
    assert got_plain == want and got_side == want
    assert plain.flush() == side.flush() == float(7 % 3)


def test_graphed_moe_forward_matches_eager(native_ops):
    """One captured CUDA graph serves any routing: replays equal eager calls bit for bit."""
    from terracemoe_simulator_b200.layer import TerracedMoE
    from terracemoe_simulator_b200.routing import TRouteConfig
    from terracemoe_simulator_b200.utils.graphs import GraphedForward
    torch.manual_seed(0)
    cfg = TRouteConfig(32, 4, 4, 2)
    layer = TerracedMoE(512, 256, 256, cfg).to(DEV, torch.bfloat16).eval()
    layer.expert_backend = "native"
    fwd = lambda t: layer(t)[0]
    x0 = torch.randn(256, 512, device=DEV, dtype=torch.bfloat16)
    graphed = GraphedForward(fwd, x0)
    for seed in range(3):
        x = torch.randn(256, 512, device=DEV, dtype=torch.bfloat16,
                        generator=torch.Generator(DEV).manual_seed(seed))
        with torch.no_grad():
            want = fwd(x)
        got = graphed(x).clone()
        assert torch.equal(got, want)
    assert graphed.replays == 3 and native_ops.take_status() == 0
    with pytest.raises(ValueError):
        graphed(torch.zeros(128, 512, device=DEV, dtype=torch.bfloat16))
    # launch-bound case: the replay is faster than the eager chain
    def timeit(f):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(50):
            f()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / 50
    with torch.no_grad():
        eager_ms = timeit(lambda: fwd(x0))
    graph_ms = timeit(lambda: graphed(x0))
    print(f"\nMoE forward, 256 tokens: eager {eager_ms * 1e3:.1f} us, graph {graph_ms * 1e3:.1f} us")
    assert graph_ms < eager_ms
