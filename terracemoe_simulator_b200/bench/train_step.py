"""End-to-end decoder training step: tokens/s through the public model API.

    python -m terracemoe_simulator_b200.bench.train_step [--steps 5 --warmup 3]
    python -m torch.distributed.run --nproc-per-node 8 \
        -m terracemoe_simulator_b200.bench.train_step --ep two_hop --rpn 2

Default shape: 16-layer decoder, d_model 2048, 16 heads, RoPE, RMSNorm, EVERY layer MoE with 64
SwiGLU experts of hidden 1024 (``--dense-ends`` restores a dense first and last layer), top-4 in
2 of 4 routing groups, one shared expert, balance aux loss coefficient 0.01, 8 sequences of 4096
tokens per GPU, bf16 parameters, AdamW; with N ranks the 4 routing groups are logical groups of
N / 4 GPUs (8 GPUs: 4 groups of 2).  One step =
pinned host -> device copy of the token batch, forward, loss, backward, gradient average of the
replicated parameters over the ranks, optimizer step, device -> host read of the loss (consumed one step later so that the host keeps
launching ahead).  With N
ranks the routed experts are sharded N ways (``--ep one_hop | two_hop``, fused peer-memory
kernels unless ``--nccl``) and every rank trains on its own sequences (weak scaling).

Timing: W warm-up steps, K timed steps between CUDA events bracketed by barrier + synchronize,
max over ranks.  Prints one JSON line on rank 0.  The reference has no such loop on GPUs; its
only training step is the CPU toy in ``tests/test_checkpoint.py:16-23``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist


def build_args(ns, world: int):
    from ..models import ModelArgs
    return ModelArgs(vocab=ns.vocab, dim=ns.dim, n_layers=ns.layers, n_heads=ns.heads,
                     seq_len=ns.seq, n_experts=ns.experts, n_groups=ns.groups, top_k=ns.top_k,
                     top_groups=ns.top_groups, d_expert=ns.d_expert, d_shared=ns.d_shared,
                     n_shared=1, dense_first=1, moe_every_layer=not ns.dense_ends,
                     balance_aux=ns.balance_aux, expert_backend=ns.backend,
                     ep_mode=ns.ep if world > 1 else "local", ep_rpn=ns.rpn,
                     ep_fused=not ns.nccl, ce_chunk=ns.ce_chunk)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--dim", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--d-expert", type=int, default=1024)
    ap.add_argument("--d-shared", type=int, default=1024)
    ap.add_argument("--groups", type=int, default=4)
    ap.add_argument("--top-k", type=int, default=4)
    ap.add_argument("--top-groups", type=int, default=2)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=8, help="sequences per GPU")
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--ep", default="two_hop", choices=["one_hop", "two_hop"])
    ap.add_argument("--rpn", type=int, default=0,
                    help="GPUs per logical group (0: world / routing groups, at least 1)")
    ap.add_argument("--dense-ends", action="store_true",
                    help="dense FFN in the first and the last layer instead of MoE everywhere")
    ap.add_argument("--balance-aux", type=float, default=0.01)
    ap.add_argument("--nccl", action="store_true", help="all_to_all arm instead of fused kernels")
    ap.add_argument("--backend", default="native", choices=["native", "grouped", "loop"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--heartbeat", action="store_true",
                    help="ranks watch each other over a TCP store and stop before the next step "
                         "when a peer left or went quiet (utils/health.py)")
    ap.add_argument("--ce-chunk", type=int, default=0,
                    help="> 0: LM head + cross-entropy in chunks of that many tokens (saves the "
                         "[tokens, vocab] logits)")
    ns = ap.parse_args(argv)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if ns.rpn <= 0:
        ns.rpn = max(world // ns.groups, 1)
    cuda = torch.cuda.is_available() and not ns.cpu
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    if cuda:
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
    else:
        device = torch.device("cpu")
    if world > 1:
        if cuda:
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
    from ..models import TerraceLM
    from ..parallel.dp import DPGradSync
    dtype = torch.bfloat16 if ns.dtype == "bf16" else torch.float32
    torch.manual_seed(1234)                      # replicated parameters start identical
    model = TerraceLM(build_args(ns, world)).to(device=device, dtype=dtype)
    if world > 1:                                # expert shards differ per rank
        g = torch.Generator(device="cpu").manual_seed(99 + rank)
        for name, p in model.named_parameters():
            if name.endswith((".w13", ".w2")) and "ffn" in name and p.dim() == 3:
                with torch.no_grad():
                    p.copy_((torch.randn(p.shape, generator=g) * p.shape[1] ** -0.5).to(p))
    sync = DPGradSync(model)
    opt = torch.optim.AdamW(model.parameters(), lr=ns.lr, weight_decay=0.1,
                            fused=True if cuda else None)
    gtok = torch.Generator(device="cpu").manual_seed(7 + rank)
    n_host = 4
    host = [torch.randint(0, ns.vocab, (ns.batch, ns.seq + 1), generator=gtok) for _ in range(n_host)]
    if cuda:
        host = [h.pin_memory() for h in host]
    model.train()
    state = {"i": 0, "loss": 0.0}

    import itertools
    from ..utils.prefetch import DeferredScalar, DevicePrefetcher
    feed = DevicePrefetcher(itertools.cycle(host), device)
    losses = DeferredScalar(device)          # every step's loss reaches the host, one step late
    health = DeferredScalar(device)          # and so does the transport's status word

    hb = None
    if ns.heartbeat and world > 1:
        from datetime import timedelta
        from ..utils.health import Heartbeat
        store = dist.TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]) + 7, world,
                              rank == 0, timeout=timedelta(seconds=60))
        hb = Heartbeat(store, rank, world, interval_s=0.5, timeout_s=30.0)

    def step():
        if hb is not None:
            hb.guard()                           # PeerLost before any launch of this step
        tok = next(feed)
        state["i"] += 1
        opt.zero_grad(set_to_none=True)
        loss, info = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        sync.sync()
        opt.step()
        prev = losses.push(loss)                 # device -> host read of the result (deferred)
        if prev is not None:
            state["loss"] = prev
        if "ep_status" in info:                  # a skipped row or a wait that ran out: stop here
            code = health.push(info["ep_status"].float().sum())
            if code:
                raise RuntimeError(f"expert-parallel kernels reported status {int(code)} "
                                   "(5: routed rows exceeded the arena's row capacity)")

    def barrier():
        if cuda:
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    for _ in range(ns.warmup):
        step()
    barrier()
    if cuda:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
    t0 = time.perf_counter()
    for _ in range(ns.steps):
        step()
    state["loss"] = losses.flush()               # the last step's loss, inside the timed region
    if cuda:
        b.record()
    barrier()
    if hb is not None:
        hb.stop()
    ms = a.elapsed_time(b) if cuda else (time.perf_counter() - t0) * 1e3
    t = torch.tensor([ms], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item() / ns.steps
    tokens = ns.batch * ns.seq * world
    status = 0
    if cuda:
        from .. import ops
        status = ops.take_status(local) if ops.custom_ops_enabled() else -1
    out = {"metric": "train_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
           "n_gpus": world, "steps": ns.steps, "warmup": ns.warmup, "ms_per_step": ms,
           "loss": state["loss"], "dtype": ns.dtype, "data": "synthetic", "scaling": "weak",
           "n_params": model.n_params(), "dp_allreduce_calls": sync.calls, "status": status,
           "config": {"model": f"decoder L{ns.layers} d{ns.dim} h{ns.heads} E{ns.experts}x{ns.d_expert} "
                               f"top{ns.top_k} M{ns.top_groups}", "global_batch": ns.batch * world,
                      "seq_len": ns.seq, "parallelism": f"ep{world}+dp{world}" if world > 1 else "single",
                      "ep_mode": ns.ep if world > 1 else "local", "rpn": ns.rpn,
                      "transport": "nccl" if ns.nccl else "fused", "optimizer": "AdamW",
                      "h2d_bytes_per_step": ns.batch * (ns.seq + 1) * 8, "d2h_bytes_per_step": 4}}
    if cuda:
        # device memory of this rank: the caching allocator's peak, and what lives outside it
        # (the peer-memory arenas of the fused transport, one per MoE layer)
        free_b, total_b = torch.cuda.mem_get_info(device)
        out["memory_gib"] = {"torch_peak": round(torch.cuda.max_memory_allocated(device) / 2 ** 30, 2),
                             "torch_reserved": round(torch.cuda.memory_reserved(device) / 2 ** 30, 2),
                             "device_in_use": round((total_b - free_b) / 2 ** 30, 2)}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
