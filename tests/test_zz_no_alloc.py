"""The allocation-free plan entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory when they need a permutation plan
(pool-managed regions, C embedders without a tensor allocator, fixed-buffer replay loops), so
``tb200_moe_plan_static`` keeps its scratch in a fixed array inside the library.  This test loads
the shared object with ctypes, calls the symbol twice in a row with different routings (the
second call meets the first call's leftovers in the shared scratch) and checks every output
against the regular entry point, which must agree exactly: the plan is integer bookkeeping plus
a permutation of the gates.  A third case sits exactly on the documented limits of the built-in
scratch (T * k = 262144 pairs, 1024 experts).
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, idx, gates, E, align):
    T, k = idx.shape
    dev = idx.device
    i32 = dict(dtype=torch.int32, device=dev)
    es, cols, pos = (torch.full((T, k), -7, **i32) for _ in range(3))
    gs = torch.full((T, k), -7.0, dtype=torch.float32, device=dev)
    seg_start, seg_count = torch.full((E,), -7, **i32), torch.full((E,), -7, **i32)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.tb200_moe_plan_static(
        ctypes.c_void_p(idx.data_ptr()), ctypes.c_void_p(gates.data_ptr()),
        ctypes.c_void_p(es.data_ptr()), ctypes.c_void_p(gs.data_ptr()),
        ctypes.c_void_p(cols.data_ptr()), ctypes.c_void_p(pos.data_ptr()),
        ctypes.c_void_p(seg_start.data_ptr()), ctypes.c_void_p(seg_count.data_ptr()),
        ctypes.c_int(T), ctypes.c_int(k), ctypes.c_int(E), ctypes.c_int(align),
        ctypes.c_void_p(stream))
    return rc, (es, gs, cols, pos, seg_start, seg_count)


def test_static_plan_matches_regular_entry_point(native_ops):
    lib = ctypes.CDLL(native_ops.status().lib)
    lib.tb200_moe_plan_static.restype = ctypes.c_int
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(5)
    for T, k, E, align in [(4096, 6, 64, 64), (1537, 4, 16, 1)]:      # two calls in a row
        idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(dev)
        gates = torch.rand(T, k, generator=g).to(dev)
        rc, got = _call_static(lib, idx, gates, E, align)
        assert rc == 0
        want = torch.ops.terrace.moe_plan(idx, gates, E, align)
        torch.cuda.synchronize()
        for name, a, b in zip(("es", "gs", "cols", "pos", "seg_start", "seg_count"), got, want):
            assert torch.equal(a, b), name


def test_static_plan_at_the_scratch_limits(native_ops):
    """T * k = 262144 and E = 1024 use the fixed array to its last word."""
    lib = ctypes.CDLL(native_ops.status().lib)
    lib.tb200_moe_plan_static.restype = ctypes.c_int
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    T, k, E = 32768, 8, 1024
    g = torch.Generator().manual_seed(9)
    # k distinct experts per token: a random start and a random odd stride around the ring
    start = torch.randint(0, E, (T, 1), generator=g)
    stride = 2 * torch.randint(0, E // 2, (T, 1), generator=g) + 1
    idx = ((start + stride * torch.arange(k)) % E).to(dev)
    gates = torch.rand(T, k, generator=g).to(dev)
    rc, got = _call_static(lib, idx, gates, E, 64)
    assert rc == 0
    want = torch.ops.terrace.moe_plan(idx, gates, E, 64)
    torch.cuda.synchronize()
    for name, a, b in zip(("es", "gs", "cols", "pos", "seg_start", "seg_count"), got, want):
        assert torch.equal(a, b), name


def test_static_plan_rejects_oversize(native_ops):
    lib = ctypes.CDLL(native_ops.status().lib)
    lib.tb200_moe_plan_static.restype = ctypes.c_int
    null = ctypes.c_void_p(0)
    rc = lib.tb200_moe_plan_static(null, null, null, null, null, null, null, null,
                                   ctypes.c_int(100000), ctypes.c_int(8), ctypes.c_int(64),
                                   ctypes.c_int(1), null)
    assert rc == 5          # TB200_ERR_SIZE: beyond the built-in scratch, nothing launched
