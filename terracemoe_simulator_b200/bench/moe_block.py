"""One MoE block (router, capacity factor, routed experts, shared expert), forward + backward.

    python -m terracemoe_simulator_b200.bench.moe_block            # DeepSeek-V3-shaped defaults
    python -m torch.distributed.run --nproc-per-node 8 \
        -m terracemoe_simulator_b200.bench.moe_block --ep two_hop --rpn 4

Defaults: d_model 7168, 256 SwiGLU experts of hidden 2048 plus one shared expert of the same
width, top-8 in 2 of 2 routing groups (quota 4), 8192 tokens per GPU, capacity factor 1.25, bf16.
With N ranks the routed experts are sharded N ways (weak scaling: tokens per GPU fixed); two-hop
groups are ``--rpn`` ranks.  The layer is the package's public ``EPTerracedMoE`` module; one step =
pinned host -> device copy of the tokens, forward, backward to every gradient, device -> host
read of the loss.  CUDA events, barrier + synchronize on both sides, max over ranks; prints one
JSON line on rank 0.  The reference has no capacity factor (drop-less only,
``terrace/layer.py:94-171``); this configuration exists for the expert-parallel block here.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--dim", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--d-expert", type=int, default=2048)
    ap.add_argument("--d-shared", type=int, default=2048)
    ap.add_argument("--groups", type=int, default=2)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--top-groups", type=int, default=2)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--capacity", type=float, default=1.25)
    ap.add_argument("--ep", default="two_hop", choices=["one_hop", "two_hop"])
    ap.add_argument("--rpn", type=int, default=0,
                    help="GPUs per logical group (0: world / routing groups, at least 1)")
    ap.add_argument("--nccl", action="store_true")
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ns = ap.parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if ns.rpn <= 0:
        ns.rpn = max(world // ns.groups, 1)
    cuda = torch.cuda.is_available() and not ns.cpu
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29543")
    device = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(local)
    if world > 1:
        if cuda:
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
    from ..parallel.moe_layer import EPTerracedMoE
    from ..routing import TRouteConfig
    dtype = torch.bfloat16 if ns.dtype == "bf16" else torch.float32
    cfg = TRouteConfig(ns.experts, ns.groups, ns.top_k, ns.top_groups)
    torch.manual_seed(1234 + rank)
    layer = EPTerracedMoE(ns.dim, ns.d_expert, ns.d_shared, cfg, n_shared=1,
                          mode=ns.ep if world > 1 else "local", rpn=ns.rpn, fused=not ns.nccl,
                          capacity_factor=ns.capacity if ns.capacity > 0 else None,
                          tokens_hint=ns.tokens).to(device=device, dtype=dtype)
    layer.train()
    g = torch.Generator(device="cpu").manual_seed(5 + rank)
    x_host = torch.randn(ns.tokens, ns.dim, generator=g).to(dtype)
    gy = torch.randn(ns.tokens, ns.dim, generator=g).to(dtype).to(device)
    if cuda:
        x_host = x_host.pin_memory()
    last = {"loss": 0.0}

    import itertools
    from ..utils.prefetch import DeferredScalar, DevicePrefetcher
    feed = DevicePrefetcher(itertools.cycle([x_host]), device)
    losses = DeferredScalar(device)

    def step():
        for p in layer.parameters():
            p.grad = None
        x = feed.take().requires_grad_(True)
        y, _ = layer(x)
        loss = (y.float() * gy.float()).mean()
        loss.backward()
        # the copy of a later input travels under this backward's weight-gradient GEMMs, where
        # the NVLink traffic pauses (a PCIe copy beside the peer-memory pushes slows them)
        feed.refill(after=layer.link_quiet_event())
        prev = losses.push(loss)
        if prev is not None:
            last["loss"] = prev

    def barrier():
        if cuda:
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    import time
    for _ in range(ns.warmup):
        step()
    barrier()
    if cuda:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
    t0 = time.perf_counter()
    for _ in range(ns.steps):
        step()
    last["loss"] = losses.flush()
    if cuda:
        b.record()
    barrier()
    ms = a.elapsed_time(b) if cuda else (time.perf_counter() - t0) * 1e3
    t = torch.tensor([ms], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item() / ns.steps
    status = 0
    if cuda:
        from .. import ops
        status = ops.take_status(local) if ops.custom_ops_enabled() else -1
    tokens = ns.tokens * world
    flops = 3 * 2 * 3 * ns.tokens * (ns.top_k * ns.d_expert + ns.d_shared) * ns.dim
    out = {"metric": "moe_block_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
           "n_gpus": world, "steps": ns.steps, "warmup": ns.warmup, "ms_per_step": ms,
           "loss": last["loss"], "dtype": ns.dtype, "data": "synthetic", "scaling": "weak",
           "status": status, "gemm_tflops_per_gpu": flops / (ms * 1e-3) / 1e12,
           "config": {"model": f"MoE block d{ns.dim} E{ns.experts}x{ns.d_expert}+shared{ns.d_shared} "
                               f"top{ns.top_k} M{ns.top_groups} cap{ns.capacity}",
                      "global_batch": tokens, "seq_len": ns.tokens,
                      "parallelism": f"ep{world}", "ep_mode": ns.ep if world > 1 else "local",
                      "rpn": ns.rpn, "transport": "nccl" if ns.nccl else "fused",
                      "h2d_bytes_per_step": x_host.numel() * x_host.element_size(),
                      "d2h_bytes_per_step": 4}}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
