"""The newest paths on one GPU, collected last and ordered from the most to the least established,
so that with ``-x`` a failure here cannot hide the suites before it.

* chunked LM head + loss in bf16 against the unchunked loss
* a flag wait that nothing satisfies: status code, then ``FusedEPContext.rebuild()``
* the scattering GEMM op alone (forward, dgrad, CTA pair; a map entry out of range)
* three token slices on three streams and arenas against the unsliced layer
* the residency protocol at toy size
"""
import os

import pytest
import torch

from test_gpu_fused_ep import _close

pytestmark = pytest.mark.gpu


def test_chunked_lm_loss_on_gpu_matches_the_unchunked_loss(native_ops):
    import torch.nn.functional as F
    from terracemoe_simulator_b200.models.decoder import chunked_lm_loss
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    n, d, v = 1000, 256, 2048
    h0 = torch.randn(n, d, device=dev).bfloat16()
    w0 = (torch.randn(v, d, device=dev) * d ** -0.5).bfloat16()
    tgt = torch.randint(0, v, (n,), device=dev)
    h1, w1 = h0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
    ref = F.cross_entropy(F.linear(h1, w1).float(), tgt)
    ref.backward()
    h2, w2 = h0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
    got = chunked_lm_loss(h2, w2, tgt, 384)                  # 1000 tokens: ragged last chunk
    got.backward()
    torch.cuda.synchronize()
    torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-4)
    _close(h2.grad.float(), h1.grad.float(), 2e-2)
    _close(w2.grad.float(), w1.grad.float(), 2e-2)


def _timeout_worker(rank, world, port, queue):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        import time
        from terracemoe_simulator_b200.parallel import fused as fz
        from terracemoe_simulator_b200.routing import TRouteConfig, t_route
        dev = torch.device("cuda", rank)
        cfg = TRouteConfig(16, 2, 4, 2)
        fctx = fz.FusedEPContext(cfg, 256, 128, 256, world=1, rank=0, rpn=1, device=dev)
        like = torch.zeros(8, device=dev)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        # wait for an arrival flag of an epoch that nothing will ever signal
        torch.ops.terrace.ep_signal(fctx.arena, fz.FK_OUT, 0, 1, 1, 0, 1 << 20, fz.FK_DATA, 0, 1,
                                    1 << 28, like)
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        status = fctx.take_status()
        # the context is still usable: after recovery a regular dispatch + combine runs clean
        g = torch.Generator().manual_seed(0)
        x = torch.randn(200, 256, generator=g).bfloat16().to(dev)
        idx, gates, _ = t_route(torch.rand(200, 16, generator=g).to(dev), torch.zeros(16, device=dev), cfg)
        fctx.rebuild()                      # recovery: tear the arena down, build a fresh one
        echo = fz.fused_dispatch_combine(fctx, x, idx, gates, mode="one_hop")
        torch.cuda.synchronize()
        err = (echo.float() - x.float()).abs().max().item()
        queue.put((rank, {"status": status, "waited": waited, "after": fctx.take_status(),
                          "echo_err": err, "epoch": fctx.epoch,
                          "canaries": len(fctx.check_canaries())}))
    except Exception as exc:  # noqa: BLE001
        import traceback
        queue.put((rank, "error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))
    finally:
        dist.destroy_process_group()


def test_flag_wait_runs_out_with_a_status_and_a_usable_context(native_ops):
    """Failure detection without a fault: a wait on a flag that nothing sets gives up after its
    limit, reports the flag-timeout code to the host, and later launches run normally."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_timeout_worker, args=(0, 1, 29791, q))
    p.start()
    try:
        item = q.get(timeout=300)
    finally:
        p.join(timeout=30)
        if p.is_alive():
            p.terminate()
    assert item[1] != "error", item[2]
    res = item[1]
    assert res["status"] == 4, res                   # ST_TIMEOUT_FLAG
    assert 1.0 < res["waited"] < 30.0, res           # the 2 s limit, not an endless spin
    assert res["after"] == 0 and res["echo_err"] < 0.2, res
    assert res["epoch"] == 1 and res["canaries"] == 0, res      # rebuilt arena, epochs restarted


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


def _pipeline_worker(rank, world, port, queue):
    import os
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        from terracemoe_simulator_b200.parallel import fused as fz
        from terracemoe_simulator_b200.routing import TRouteConfig, t_route
        dev = torch.device("cuda", rank)
        E, k, H, d, T = 16, 4, 256, 128, 1000
        cfg = TRouteConfig(E, 2, k, 1)
        g = torch.Generator().manual_seed(5)
        w13 = (torch.randn(E, H, 2 * d, generator=g) * H ** -0.5).bfloat16().to(dev)
        w2 = (torch.randn(E, d, H, generator=g) * d ** -0.5).bfloat16().to(dev)
        x0 = torch.randn(T, H, generator=g).bfloat16().to(dev)
        gy = torch.randn(T, H, generator=g).bfloat16().to(dev)
        idx, gates0, _ = t_route(torch.rand(T, E, generator=g).to(dev), torch.zeros(E, device=dev), cfg)
        plain = fz.FusedEPContext(cfg, H, d, T, world=1, rank=0, rpn=1, device=dev)
        pipe = fz.PipelinedFusedEP(cfg, H, d, T, n=3, world=1, rank=0, rpn=1, device=dev)
        res = {}
        for name, ctx in (("plain", plain), ("pipe", pipe)):
            x = x0.clone().requires_grad_(True)
            gates = gates0.clone().requires_grad_(True)
            a, b = w13.clone().requires_grad_(True), w2.clone().requires_grad_(True)
            for _ in range(2):                       # twice: buffers and streams are reused
                for t in (x, gates, a, b):
                    t.grad = None
                y = fz.run_fused(ctx, x, idx, gates, a, b, mode="one_hop")
                y.backward(gy)
            torch.cuda.synchronize()
            res[name] = [t.detach().float().cpu() for t in (y, x.grad, gates.grad, a.grad, b.grad)]
        queue.put((rank, res, plain.take_status() or pipe.take_status(),
                   len(plain.check_canaries()) + len(pipe.check_canaries())))
    except Exception as exc:  # noqa: BLE001
        import traceback
        queue.put((rank, "error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))
    finally:
        dist.destroy_process_group()


def test_token_pipeline_on_one_gpu_equals_the_unsliced_layer(native_ops):
    """Three token slices on three streams and arenas against the unsliced layer: outputs, input
    and gate gradients are bit-equal (a row's products do not depend on its tile), weight
    gradients are sums of three partial results and agree within rounding."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_pipeline_worker, args=(0, 1, 29811, q))
    p.start()
    try:
        item = q.get(timeout=300)
    finally:
        p.join(timeout=30)
        if p.is_alive():
            p.terminate()
    assert item[1] != "error", item[2]
    _, res, status, canaries = item
    assert status == 0 and canaries == 0
    for i in (0, 1):
        assert torch.equal(res["plain"][i], res["pipe"][i])
    _close(res["pipe"][2], res["plain"][2], 1e-2)        # gate gradients: lane partition differs
    for i in (3, 4):
        _close(res["pipe"][i], res["plain"][i], 2e-2)


def test_residency_protocol_runs_and_returns_a_measured_profile(native_ops):
    """The memory protocol at toy size: four (layers, tokens) points, a fitted activation slope
    and an overhead share that make physical sense."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, TERRACE_CUSTOM_OPS="1", PYTHONPATH=root)
    proc = subprocess.run([sys.executable, "-m", "terracemoe_simulator_b200.bench.residency",
                           "--layers", "3", "5", "--batch", "1", "2", "--seq", "256", "--dim", "256",
                           "--experts", "8", "--d-expert", "128"],
                          env=env, capture_output=True, timeout=900, cwd=root)
    assert proc.returncode == 0, proc.stderr.decode(errors="replace")[-3000:]
    out = json.loads([l for l in proc.stdout.decode().splitlines() if l.startswith("{")][-1])
    prof = out["profile"]
    assert prof["measured"] is True and len(out["samples"]) == 4
    assert prof["activation_bytes_per_token_layer"] > 0          # deeper and longer costs memory
    assert 0.0 <= prof["overhead_frac"] < 0.5
    peaks = [s["peak_allocated"] for s in out["samples"]]
    assert max(peaks) > min(peaks)
