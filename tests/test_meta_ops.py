"""Shape-only (Meta) implementations of the native ops: every tensor-returning op answers on
``device="meta"`` with the shapes and dtypes its CUDA kernel produces, and the decoder runs its
forward pass through the native-op path under ``FakeTensorMode`` on a host without a GPU."""
import os

import pytest
import torch

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                   "terracemoe_simulator_b200", "ops", "lib", "terrace_b200_ops.so")
pytestmark = pytest.mark.skipif(not os.path.isfile(LIB), reason="native library not built")


@pytest.fixture()
def lib(monkeypatch):
    monkeypatch.setenv("TERRACE_CUSTOM_OPS", "1")
    from terracemoe_simulator_b200 import ops
    ops.reset()
    assert ops.status().loaded, ops.status().reason
    yield torch.ops.terrace
    monkeypatch.undo()
    ops.reset()


def _m(*shape, dtype=torch.bfloat16):
    return torch.empty(*shape, device="meta", dtype=dtype)


def _sig(ts):
    ts = ts if isinstance(ts, (tuple, list)) else (ts,)
    return [(tuple(t.shape), t.dtype) for t in ts]


def test_compute_ops_answer_on_meta(lib):
    bf, f32, i32, i64 = torch.bfloat16, torch.float32, torch.int32, torch.int64
    T, H, E, k, M, d = 40, 64, 16, 4, 2, 32
    x, w = _m(T, H), _m(H)
    assert _sig(lib.rmsnorm_fwd(x, w, 1e-5)) == [((T, H), bf), ((T,), f32)]
    dx, part = lib.rmsnorm_bwd(x, w, x, _m(T, dtype=f32))
    assert dx.shape == (T, H) and part.shape[1] == H and part.dtype == f32
    route = [((T, k), i64), ((T, k), f32), ((T, M), i64), ((E,), f32), ((T, k), f32)]
    assert _sig(lib.route_select(_m(T, E, dtype=f32), _m(E, dtype=f32), 4, k, M, 2)) == route
    assert _sig(lib.route_fused(x, _m(E, H), _m(E, dtype=f32), 4, k, M, 2)) == route
    assert _sig(lib.route_select_bwd(_m(T, k, dtype=f32), _m(T, k, dtype=f32), _m(T, k, dtype=f32),
                                     _m(T, k, dtype=i64), E)) == [((T, E), f32)]
    plan = lib.moe_plan(_m(T, k, dtype=i64), _m(T, k, dtype=f32), E, 64)
    assert _sig(plan) == [((T, k), i32), ((T, k), f32), ((T, k), i32), ((T, k), i32), ((E,), i32),
                          ((E,), i32)]
    rows = T * k + E * 63
    xs = lib.moe_scatter_rows(x, plan[3], rows)
    assert _sig(xs) == [((rows, H), bf)]
    w13, w2 = _m(E, H, 2 * d), _m(E, d, H)
    act, h13 = lib.grouped_gemm(xs, w13, plan[4], plan[5], 0, 1, True, 0, 64)
    assert _sig([act, h13]) == [((rows, d), bf), ((rows, 2 * d), bf)]
    out, none = lib.grouped_gemm(act, w2, plan[4], plan[5], 0, 0, False, 0, 64)
    assert out.shape == (rows, H) and none.numel() == 0
    assert lib.grouped_gemm(out, w2, plan[4], plan[5], 1, 0, False, 0, 64)[0].shape == (rows, d)
    assert _sig(lib.moe_combine(out, plan[3], plan[0], plan[1], 4)) == [((T, H), bf)]
    dout, dgs = lib.moe_combine_bwd(x, out, plan[3], plan[1], True)
    assert dout.shape == out.shape and _sig(dgs) == [((T, k), f32)]
    assert _sig(lib.swiglu_bwd(h13, act)) == [((rows, 2 * d), bf)]
    assert _sig(lib.grouped_wgrad(xs, h13, plan[4], plan[5], 0, 64)) == [((E, H, 2 * d), bf)]
    assert lib.zero_pad_rows(xs, plan[4], plan[5], 64) is None
    assert lib.grouped_wgrad_out(xs, h13, _m(E, H, 2 * d), 0, plan[4], plan[5], 0, 64) is None
    q = _m(2, 4, 128, 64)
    assert _sig(lib.attn_fwd(q, q, q, True, 0.125)) == [((2, 4, 128, 64), bf), ((2, 4, 128), f32)]
    assert _sig(lib.attn_bwd(q, q, q, q, q, _m(2, 4, 128, dtype=f32), True, 0.125)) == \
        [((2, 4, 128, 64), bf)] * 3


def test_transport_ops_answer_on_meta(lib):
    i32, f32, i64 = torch.int32, torch.float32, torch.int64
    world, E, k, M, T, H = 4, 16, 4, 2, 24, 64
    arena = lib.symm_make_arena([0] * world, [16 * i for i in range(12)],
                                [world, 1, E, E // world, 2, 2, T, k, M, k // M, H, 512])
    es, gs, cols, rank_local, hist = lib.ep_plan_pass1(_m(T, k, dtype=i64), _m(T, k, dtype=f32), E)
    assert _sig([es, gs, hist]) == [((T, k), i32), ((T, k), f32), ((128, E), i32)]
    assert _sig(lib.ep_plan(arena, hist, None, 1, 64)) == \
        [((E,), i32), ((E // world,), i32), ((E // world,), i32), ((world, 2), i32), ((E,), i32)]
    ranka, chunka = lib.hopa_rank(arena, es)
    assert _sig([ranka, chunka]) == [((T, M), i32), ((128, 2), i32)]
    x = _m(T, H)
    pos, rowa = lib.hopa_push(arena, x, es, gs, rank_local, hist, _m(E, dtype=i32), ranka, chunka,
                              None, 4, True, 1, 1, _m(1, dtype=i32))
    assert _sig([pos, rowa]) == [((T, k), i32), ((T, M), i32)]
    assert _sig(lib.ep_pull_combine(arena, pos, es, gs, 0, 4, 3, 1, 0)) == [((T, H), torch.bfloat16)]
    assert _sig(lib.origin_combine(arena, es, rowa, 5, 4, 1, False)) == [((T, H), torch.bfloat16)]
    assert _sig(lib.origin_pull_dgate(arena, es, rowa, 7, 1)) == [((T, k), f32)]
    assert lib.ep_push(arena, x, es, rank_local, hist, _m(E, dtype=i32), None, pos, None, 0, 0,
                       False, 2, 31, 0, E // world, _m(1, dtype=i32), -1, T * k) is None


def test_decoder_forward_runs_through_the_native_ops_on_fake_tensors(lib):
    """FakeTensorMode with fake CUDA tensors on a host that may have no GPU: the model takes the
    native-op path (its live counters move) and returns a scalar loss of the right kind.  (The
    backward pass needs a CUDA context for the autograd engine and is covered by the GPU tests.)"""
    from torch._subclasses.fake_tensor import FakeTensorMode
    from terracemoe_simulator_b200.models import ModelArgs, TerraceLM
    from terracemoe_simulator_b200.ops import native
    args = ModelArgs(vocab=512, dim=256, n_layers=3, n_heads=4, seq_len=128, n_experts=16,
                     n_groups=4, top_k=4, top_groups=2, d_expert=128, d_shared=256,
                     expert_backend="native", dense_first=1)
    before = dict(native.LIVE)
    default = torch.get_default_dtype()
    try:
        with FakeTensorMode():
            torch.set_default_dtype(torch.bfloat16)
            with torch.device("cuda"):
                model = TerraceLM(args)
            ids = torch.randint(0, 512, (4, 128), device="cuda")
            loss, _info = model(ids, ids)
            assert loss.shape == () and loss.device.type == "cuda"
    finally:
        torch.set_default_dtype(default)
    for name in ("rmsnorm", "moe_experts_local", "attention", "linear"):
        assert native.LIVE[name] > before[name], name
    assert native.LIVE["route_fused"] > before["route_fused"]
