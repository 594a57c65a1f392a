"""Shared measurement protocol of the probe scripts in this package.

Every probe runs one process per device under ``python -m torch.distributed.run`` (NCCL on
GPUs; ``--cpu`` or a machine without CUDA selects gloo, which is how the test suite exercises
the plumbing).  Times are taken on the device with CUDA events on the launching stream (host
``perf_counter`` on CPU) and reduced with MAX over the ranks, because a collective ends when
its last participant ends.

Two timing styles, the same two the reference's probes use (``bench/a2a_form_probe.py:56-77``):

``burst``    n calls back to back, one synchronisation at the end, cost = total / n;
``percall``  ranks aligned on a barrier, then one call timed on its own, median of n.
"""
from __future__ import annotations

import json
import os
import statistics
import time
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class Env:
    rank: int
    world: int
    local: int
    device: torch.device
    cuda: bool


def init(cpu: bool = False) -> Env:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29631")
    cuda = torch.cuda.is_available() and not cpu
    if cuda:
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    else:
        device = torch.device("cpu")
        dist.init_process_group("gloo", rank=rank, world_size=world)
    return Env(rank, world, local, device, cuda)


def finish(env: Env) -> None:
    dist.barrier()
    dist.destroy_process_group()


def sync(env: Env) -> None:
    if env.cuda:
        torch.cuda.synchronize()


def max_over_ranks(env: Env, ms: float, group=None) -> float:
    t = torch.tensor([ms], dtype=torch.float32, device=env.device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def _elapsed_ms(env: Env, fn, n: int) -> float:
    """Milliseconds for n back-to-back calls of fn, measured on this rank's device."""
    if env.cuda:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)
    t0 = time.perf_counter()
    for _ in range(n):
        fn()
    return (time.perf_counter() - t0) * 1e3


def burst(env: Env, fn, n: int, group=None) -> float:
    dist.barrier()
    sync(env)
    return max_over_ranks(env, _elapsed_ms(env, fn, n) / n, group)


def percall(env: Env, fn, n: int, group=None) -> float:
    out = []
    for _ in range(n):
        dist.barrier()
        sync(env)
        out.append(max_over_ranks(env, _elapsed_ms(env, fn, 1), group))
    return statistics.median(out)


def spread(xs) -> float:
    return (max(xs) - min(xs)) / max(min(xs), 1e-12)


def median_of(env: Env, style, fn, n: int, repeats: int, group=None):
    xs = [style(env, fn, n, group) for _ in range(repeats)]
    return statistics.median(xs), spread(xs)


def write_json(env: Env, path: str, payload: dict) -> None:
    if env.rank == 0:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w", encoding="utf-8") as fh:
            json.dump(payload, fh, indent=1)
        print(f"wrote {path}", flush=True)


def say(env: Env, text: str) -> None:
    if env.rank == 0:
        print(text, flush=True)
