"""Data-parallel gradient sync and the decoder training-step benchmark on gloo ranks."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from terracemoe_simulator_b200.models import ModelArgs, TerraceLM
        from terracemoe_simulator_b200.parallel.dp import DPGradSync
        torch.manual_seed(0)
        a = ModelArgs(vocab=50, dim=32, n_layers=3, n_heads=2, seq_len=16, n_experts=8, n_groups=2,
                      top_k=2, top_groups=1, d_expert=16, d_shared=16, ep_mode="one_hop")
        model = TerraceLM(a)
        sync = DPGradSync(model, bucket_mb=0.01)          # tiny buckets: several all-reduces
        g = torch.Generator().manual_seed(10 + rank)
        tok = torch.randint(0, 50, (2, 17), generator=g)
        loss, _ = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        before = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
        sync.sync()
        after = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
        rep = [n for n, _ in sync.replicated]
        shard = [n for n, _ in sync.sharded]
        queue.put((rank, {n: before[n].numpy() for n in before}, {n: after[n].numpy() for n in after},
                   rep, shard, sync.calls, len(sync.buckets)))
        dist.barrier()
    except Exception as exc:  # noqa: BLE001
        import traceback
        queue.put((rank, "error", f"{exc}\n{traceback.format_exc()}"))
    finally:
        dist.destroy_process_group()


def test_dp_sync_averages_replicated_and_leaves_expert_shards():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, 29881, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for item in out:
        assert item[1] != "error", item[2]
    out.sort(key=lambda t: t[0])
    (_, b0, a0, rep, shard, calls, n_buckets), (_, b1, a1, _, _, _, _) = out
    assert shard and all(n.endswith((".w13", ".w2")) for n in shard)
    assert calls == n_buckets > 1
    for n in rep:
        if n not in b0:
            continue
        np.testing.assert_allclose(a0[n], (b0[n] + b1[n]) / 2, rtol=1e-5, atol=1e-7)
        np.testing.assert_array_equal(a0[n], a1[n])
    for n in shard:
        np.testing.assert_array_equal(a0[n], b0[n])         # untouched
        np.testing.assert_array_equal(a1[n], b1[n])


def test_is_expert_sharded_only_for_ep_layers():
    from terracemoe_simulator_b200.models import ModelArgs, TerraceLM
    from terracemoe_simulator_b200.parallel.dp import DPGradSync
    a = ModelArgs(vocab=50, dim=32, n_layers=3, n_heads=2, seq_len=16, n_experts=8, n_groups=2,
                  top_k=2, top_groups=1, d_expert=16, d_shared=16)
    sync = DPGradSync(TerraceLM(a))                       # local experts: everything replicated
    assert not sync.sharded and sync.world == 1
    sync.sync()                                           # no-op without a process group
    assert sync.calls == 0


@pytest.mark.parametrize("nproc,extra", [(1, ["--backend", "grouped"]),
                                         (2, ["--nccl", "--ep", "two_hop", "--heartbeat",
                                              "--ce-chunk", "24"])])
def test_train_step_bench_runs_on_cpu(nproc, extra):
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(29885 + nproc),
           "-m", "terracemoe_simulator_b200.bench.train_step", "--cpu", "--dtype", "fp32",
           "--layers", "3", "--dim", "64", "--heads", "4", "--experts", "8", "--d-expert", "32",
           "--d-shared", "32", "--groups", "2", "--top-k", "4", "--seq", "32", "--batch", "2",
           "--vocab", "100", "--steps", "2", "--warmup", "1"] + extra
    proc = subprocess.run(cmd, capture_output=True, env=env, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr.decode(errors="replace")[-3000:]
    line = [l for l in proc.stdout.decode().splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert out["n_gpus"] == nproc and out["value"] > 0 and np.isfinite(out["loss"])
    assert out["config"]["parallelism"] == ("single" if nproc == 1 else "ep2+dp2")
    if nproc == 2:
        assert out["dp_allreduce_calls"] >= 3


@pytest.mark.parametrize("nproc,extra", [(1, []), (2, ["--nccl", "--ep", "two_hop"])])
def test_moe_block_bench_runs_on_cpu(nproc, extra):
    """The V3-shaped block benchmark (capacity factor, shared expert) at toy size, 1 and 2 ranks."""
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(29895 + nproc),
           "-m", "terracemoe_simulator_b200.bench.moe_block", "--cpu", "--dtype", "fp32",
           "--dim", "64", "--experts", "8", "--d-expert", "32", "--d-shared", "32", "--groups", "2",
           "--top-k", "4", "--top-groups", "2", "--tokens", "64", "--capacity", "1.25",
           "--steps", "2", "--warmup", "1"] + extra
    proc = subprocess.run(cmd, capture_output=True, env=env, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr.decode(errors="replace")[-3000:]
    line = [l for l in proc.stdout.decode().splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert out["n_gpus"] == nproc and out["value"] > 0 and out["ms_per_step"] > 0
