"""Opt-in transport variants on one GPU; collected last so that the established suites run first.

World 1 exercises the whole mechanism of the scattering GEMM epilogue on a single device: the
push writes the row map, the second expert GEMM (and the last dgrad GEMM) store every output row
through a per-row destination into the return slots, and the combine reduces from those slots.
The destinations are this GPU's own memory here; with more GPUs only the base addresses change
(``tests/test_gpu_fused_ep.py::test_epilogue_push_world2_equals_two_hop_pull``, opt-in).
"""
import pytest
import torch

from test_gpu_fused_ep import _close, _run

pytestmark = pytest.mark.gpu


def test_epilogue_push_world1_equals_local_kernels(native_ops, monkeypatch):
    """Bit-equal to the local kernels: same GEMM tiles, same reduction order, different route."""
    monkeypatch.setenv("TERRACE_EP_EPILOGUE_PUSH", "1")
    (rank, res, echo, x0, status, live), = _run(1, 1, 29781)
    assert status == 0
    assert live["epilogue_push_fwd"] == 1 and live["epilogue_push_bwd"] == 1
    for i, (a, b) in enumerate(zip(res["one_hop"], res["ref"])):
        if i == 2:      # gate gradients: same dot products, different lane partition
            _close(a, b, 1e-2)
        else:
            assert torch.equal(a, b)
    _close(echo, x0, 2e-2)


@pytest.mark.parametrize("mode,pair", [(0, "0"), (1, "0"), (0, "1")])
def test_gemm_scatter_epilogue_equals_plain_kernel_plus_permutation(native_ops, mode, pair):
    """The GEMM alone: rows leave through a random permutation into a second buffer; a map entry
    outside the buffers is skipped and reported (status 5), never stored."""
    import os
    import subprocess
    import sys
    code = f"""
import torch
from terracemoe_simulator_b200 import ops
from terracemoe_simulator_b200.ops import native
assert ops.custom_ops_enabled()
lib = torch.ops.terrace
torch.manual_seed(0)
dev, bf = "cuda", torch.bfloat16
E, K, N, mode = 4, 256, 512, {mode}
cnt = torch.tensor([300, 0, 129, 1024], dtype=torch.int32, device=dev)
pad = (cnt + 63) // 64 * 64
st = (torch.cumsum(pad, 0) - pad).to(torch.int32)
rows = int(pad.sum())
A = torch.randn(rows, K, device=dev, dtype=bf)
W = (torch.randn(E, K, N, device=dev, dtype=bf) if mode == 0
     else torch.randn(E, N, K, device=dev, dtype=bf)) * K ** -0.5
real = torch.cat([torch.arange(int(s), int(s) + int(c), device=dev) for s, c in zip(st, cnt)])
slots = 2048
perm = torch.randperm(2 * slots, device=dev)[:real.numel()]          # two destination buffers
row_map = torch.full((rows,), -1, dtype=torch.int32, device=dev)
row_map[real] = perm.to(torch.int32)
ret = torch.zeros(2, slots, N, device=dev, dtype=bf)
base = torch.tensor([ret[0].data_ptr(), ret[1].data_ptr()], dtype=torch.int64, device=dev)
lib.grouped_gemm_scatter(A, W, st, cnt, mode, row_map, base, slots)
plain = lib.grouped_gemm(A, W, st, cnt, mode, 0, False, 0, 0)[0]
want = torch.zeros_like(ret).view(2 * slots, N)
want[perm] = plain[real]
torch.cuda.synchronize()
assert torch.equal(ret.view(2 * slots, N), want), (ret.float().view(-1, N) - want.float()).abs().max()
assert native.take_status(0) == 0
# one map entry points outside both buffers: skipped, reported
row_map[real[5]] = 2 * slots + 7
ret.zero_()
lib.grouped_gemm_scatter(A, W, st, cnt, mode, row_map, base, slots)
torch.cuda.synchronize()
want[perm[5]] = 0
assert torch.equal(ret.view(2 * slots, N), want)
assert native.take_status(0) == 5
print("ok")
"""
    env = dict(os.environ, TERRACE_CUSTOM_OPS="1", TERRACE_GEMM_PAIR=pair)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    proc = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, timeout=600)
    assert proc.returncode == 0 and b"ok" in proc.stdout, proc.stderr.decode(errors="replace")[-3000:]
