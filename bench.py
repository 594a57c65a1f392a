#!/usr/bin/env python
"""Headline benchmark: MoE-layer tokens/s (forward + backward) and dispatch+combine time on the
single-MoE-layer configuration (bf16, d_model 4096, 64 SwiGLU experts of hidden 1408, top-6,
4 routing groups, M = 2, 4096 tokens per GPU, x ~ N(0,1), router W ~ N(0, 0.02)).

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference]

For N > 1 it is launched under ``python -m torch.distributed.run`` (one rank per GPU, NCCL).
Per-GPU work is fixed as N grows (weak scaling): 4096 tokens per GPU, 64 experts in total
spread over the N GPUs.  Logical two-hop groups: N=8 -> 4 groups of 2 GPUs, N=4 -> 4 groups of
1, N=2 -> 2 groups of 1; N=1 runs the experts locally.  One step = router + routed experts
(dispatch, grouped SwiGLU GEMMs, combine), forward and backward down to the gradients of x, the
router weight and both expert weights.  Both the one-hop and the two-hop path are timed; the
headline value is the faster of the two and ``config.path`` names it.

Timing: CUDA events on the launching stream, max over ranks, barrier + synchronize on both
sides; the 2.2 GB of expert weights per step exceed the 126 MB L2, so no L2 flush is needed.
The block of K steps is repeated ``--repeats`` times (default 5) and the median block is the
reported one (minimum and maximum beside it); SM clocks are sampled over all timed blocks.
Before any timing, one step on a 512-token slice checks every path (``parity``): one-hop against
two-hop bit for bit, and outputs and all gradients against a dense fp32 PyTorch oracle.  A path
that fails the check is reported and not used for the headline.  With more than one GPU the
remote-read schedule (``TERRACE_EP_OVERLAP=0``) is timed beside the default overlap schedule as
the A/B arm (``paths.*_pull``).
The ``e2e`` entry repeats the measurement through the public API with a pinned-host -> device
copy of every step's tokens (on a side stream, two steps ahead, by the package's
``DevicePrefetcher``; each copy starts where the previous backward's NVLink traffic pauses,
``FusedEPContext.link_quiet_event``, because a PCIe copy beside the peer-memory pushes slows
them) and a device -> host read of every step's loss inside the timed region
(``DeferredScalar``: a non-blocking copy to pinned memory, consumed three steps later, so the host
keeps launching ahead of the device; the last value is read before the closing synchronize).
``--impl reference`` runs the unmodified reference (``baseline/_ref``: a plain copy of its
``terrace`` package, it has no build system to install) through ``ep_moe_forward`` /
``ta2a_moe_forward`` on NCCL for the same configuration.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))

D_MODEL, N_EXPERTS, D_EXPERT, TOP_K, TOP_GROUPS, TOKENS = 4096, 64, 1408, 6, 2, 4096
ROUTING_GROUPS = {1: 4, 2: 2, 4: 4, 8: 4}
RPN = {1: 1, 2: 1, 4: 1, 8: 2}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.lines.append(line.strip())
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def setup_dist(n_gpus: int, force: bool):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    if world > 1 or force:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", local))
    return rank, world, local


def timed(fn, steps: int, warmup: int, world: int, repeats: int = 1, drain=None):
    """W warm-up steps, then ``repeats`` blocks of exactly K steps, each between CUDA events with
    a barrier + synchronize on both sides; returns the max-over-ranks ms of every block.
    ``drain`` (optional) runs after the last step of a block and before its closing event:
    deferred device-to-host reads are completed inside the timed region."""
    import torch
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    blocks, host = [], []
    for _ in range(repeats):
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        h0 = time.perf_counter()
        for _ in range(steps):
            fn()
        host.append((time.perf_counter() - h0) * 1e3 / steps)     # enqueue time, no sync inside
        if drain is not None:
            drain()
        t1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = torch.tensor([t0.elapsed_time(t1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        blocks.append(ms.item())
    # host time to enqueue one step (this rank, median block): close to the device time per step
    # means the launch queue runs dry and the step is bound by the host
    timed.host_ms_per_step = statistics.median(host) if host else None
    return blocks


def block_stats(blocks, steps):
    per = sorted(b / steps for b in blocks)
    return {"ms_per_step": statistics.median(per), "ms_min": per[0], "ms_max": per[-1],
            "blocks": len(per)}


def make_problem(rank: int, world: int, device):
    import torch
    g = torch.Generator(device="cpu").manual_seed(1234)
    router_w = (torch.randn(N_EXPERTS, D_MODEL, generator=g) * 0.02)
    epr = N_EXPERTS // world
    # every rank draws the full weight stream so shards are consistent, keeps only its own
    w13_shard = w2_shard = None
    for r in range(world):
        a = torch.randn(epr, D_MODEL, 2 * D_EXPERT, generator=g) * D_MODEL ** -0.5
        b = torch.randn(epr, D_EXPERT, D_MODEL, generator=g) * D_EXPERT ** -0.5
        if r == rank:
            w13_shard, w2_shard = a, b
    gx = torch.Generator(device="cpu").manual_seed(100 + rank)
    x_host = torch.randn(TOKENS, D_MODEL, generator=gx).bfloat16().pin_memory()
    gy = torch.randn(TOKENS, D_MODEL, generator=gx).bfloat16().to(device)
    return (router_w.bfloat16().to(device), w13_shard.bfloat16().to(device),
            w2_shard.bfloat16().to(device), x_host, gy)


PARITY_TOKENS = 512
PARITY_TOL = 5e-2        # relative to the largest magnitude of the oracle tensor (bf16 pipeline)


def fp32_oracle(rank, world, x, idx, gates, gy, w13, w2):
    """Dense fp32 PyTorch restatement of the routed experts over all ranks' tokens and all
    experts; returns this rank's (y, dx, dgates, dw13, dw2)."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    def gather(t):
        if world == 1:
            return t
        out = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(out, t.contiguous())
        return torch.cat(out)
    T = x.shape[0]
    xa = gather(x).float().requires_grad_(True)
    ga = gather(gates.float()).requires_grad_(True)
    ia, gya = gather(idx), gather(gy).float()
    w13a, w2a = gather(w13.detach()), gather(w2.detach())        # bf16, all experts
    epr = w13.shape[0]
    y = torch.zeros_like(xa)
    dw13 = torch.zeros(epr, *w13.shape[1:], device=x.device)
    dw2 = torch.zeros(epr, *w2.shape[1:], device=x.device)
    own = []
    for e in range(w13a.shape[0]):
        tok, col = (ia == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        mine = e // epr == rank
        a = w13a[e].float().requires_grad_(mine)
        b = w2a[e].float().requires_grad_(mine)
        g, u = (xa[tok] @ a).chunk(2, dim=-1)
        y = y.index_add(0, tok, ga[tok, col].unsqueeze(1) * ((F.silu(g) * u) @ b))
        if mine:
            own.append((e - rank * epr, a, b))
    y.backward(gya)
    for le, a, b in own:
        dw13[le], dw2[le] = a.grad, b.grad
    lo = rank * T
    return [y.detach()[lo:lo + T], xa.grad[lo:lo + T], ga.grad[lo:lo + T], dw13, dw2]


def parity_check(runners, cfg, rank, world, x_dev, gy, router_w, w13, w2):
    """One forward + backward of every path on a 512-token slice, outside any timed region."""
    import torch
    import torch.distributed as dist
    from terracemoe_simulator_b200.ops import native
    from terracemoe_simulator_b200.parallel.moe_layer import _route, routed_experts
    n = PARITY_TOKENS
    x0, g0 = x_dev.detach()[:n].contiguous(), gy[:n].contiguous()
    with torch.no_grad():
        idx, gates0, _, _ = _route(x0, router_w.detach(), next(iter(runners.values())).bias, cfg)
    got = {}
    for name, r in runners.items():
        x = x0.clone().requires_grad_(True)
        gates = gates0.clone().float().requires_grad_(True)
        a, b = w13.detach().clone().requires_grad_(True), w2.detach().clone().requires_grad_(True)
        y = routed_experts(x, idx, gates, a, b, cfg, mode=r.mode, world=world, rpn=r.rpn,
                           fused=r.fused, ctx=r.ctx)
        y.backward(g0)
        got[name] = [t.detach().float() for t in (y, x.grad, gates.grad, a.grad, b.grad)]
    torch.cuda.synchronize()
    status = native.take_status(torch.cuda.current_device())
    oracle = fp32_oracle(rank, world, x0, idx, gates0, g0, w13, w2)
    report = {"tokens": n, "status": status, "paths": {}}
    names = list(got)
    flags = torch.zeros(len(names) + 1, device=x0.device)
    for i, name in enumerate(names):
        err = max(((a - b.float()).abs().max() / (b.float().abs().max() + 1e-12)).item()
                  for a, b in zip(got[name], oracle))
        flags[i] = err
    hops = [n_ for n_ in names if n_ in ("one_hop", "two_hop", "one_hop_pull", "two_hop_pull")]
    same = all(torch.equal(a, b) for n_ in hops[1:] for a, b in zip(got[hops[0]], got[n_]))
    flags[-1] = 0.0 if same else 1.0
    if world > 1:
        dist.all_reduce(flags, op=dist.ReduceOp.MAX)
    for i, name in enumerate(names):
        report["paths"][name] = {"max_rel_err_vs_fp32": flags[i].item(),
                                 "ok": bool(flags[i].item() < PARITY_TOL)}
    report["max_rel_err_vs_fp32"] = max(flags[:-1]).item()
    report["one_hop_eq_two_hop"] = bool(flags[-1].item() == 0.0) if len(hops) > 1 else None
    if world > 1:
        st = torch.tensor([float(status)], device=x0.device)
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
        report["status"] = int(st.item())
    return report


def run_ours(args, rank, world, local):
    import torch
    sys.path.insert(0, ROOT)
    from terracemoe_simulator_b200 import ops
    from terracemoe_simulator_b200.ops import native
    from terracemoe_simulator_b200.parallel import fused as fz
    from terracemoe_simulator_b200.parallel.moe_layer import MoELayerRunner
    from terracemoe_simulator_b200.routing import TRouteConfig

    assert ops.custom_ops_enabled(), "native library missing: run __graft_entry__.build()"
    device = torch.device("cuda", local)
    router_w, w13, w2, x_host, gy = make_problem(rank, world, device)
    cfg = TRouteConfig(N_EXPERTS, ROUTING_GROUPS[world], TOP_K, TOP_GROUPS)
    params = [t.requires_grad_(True) for t in (router_w, w13, w2)]
    runners = {}
    if world == 1:
        variants = [("local", "local", None)]
    else:
        variants = [("one_hop", "one_hop", None), ("two_hop", "two_hop", None)]
        if not args.nccl_arm and not args.no_ab and fz.flag_bool("TERRACE_EP_OVERLAP", True):
            variants += [("one_hop_pull", "one_hop", False), ("two_hop_pull", "two_hop", False)]
    for name, mode, overlap in variants:
        runners[name] = MoELayerRunner(cfg, D_MODEL, D_EXPERT, TOKENS, world=world, rank=rank,
                                       rpn=RPN[world], mode=mode, fused=not args.nccl_arm,
                                       device=device, overlap=overlap)
    x_dev = x_host.to(device).requires_grad_(True)
    gy_flat, inv_n = gy.reshape(-1), 1.0 / gy.numel()
    if args.no_parity:       # profiling runs: keep the launch stream to the steps themselves
        parity = {"skipped": True, "paths": {n: {"ok": True} for n in runners}}
    else:
        parity = parity_check(runners, cfg, rank, world, x_dev, gy, router_w, w13, w2)
    # end-to-end path: every step's tokens come from pinned host memory through the package's
    # input prefetcher (the copy of step i+1 runs on a side stream during step i)
    import itertools
    from terracemoe_simulator_b200.utils.prefetch import DeferredScalar, DevicePrefetcher
    host_batches = [x_host] + [x_host.clone().pin_memory() for _ in range(2)]
    feed = DevicePrefetcher(itertools.cycle(host_batches), device)
    variant = args.e2e_variant
    # every step's loss is read on the host, 3 steps late
    losses = DeferredScalar(device, lag=3)

    def make_step(path, e2e: bool):
        runner = runners[path]
        quiet = getattr(getattr(runner, "ctx", None), "link_quiet_event", lambda: None)

        def step():
            for p in params:
                p.grad = None
            if not e2e or variant == "no_h2d":
                x = x_dev
                x.grad = None
            elif variant == "ungated":
                x = next(feed).requires_grad_(True)         # takes a batch, starts the next copy
            else:
                x = feed.take().requires_grad_(True)
            y = runner(x, *params)
            if e2e:
                loss = torch.dot(y.reshape(-1).to(gy_flat.dtype), gy_flat) * inv_n   # one reduction
                loss.backward()
                if variant in ("default", "no_read"):
                    # A PCIe copy that runs beside the peer-memory pushes slows them (measured:
                    # +0.35 ms per step on 4 GPUs).  The copy of a later input therefore waits
                    # for the point of this backward where the NVLink traffic pauses -- the
                    # weight-gradient GEMMs -- and travels under them.
                    feed.refill(after=quiet())
                if variant == "no_read":
                    return None
                return losses.push(loss)     # device -> host read of the result, a few steps late
            y.backward(gy)
            return None
        return step

    results = {}
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()          # polls through the warm-ups and every timed block of every path
    from terracemoe_simulator_b200.utils import trace
    if trace.enabled():
        trace.report(group=True if world > 1 else None)      # drop the parity step's spans
    for path in runners:
        native.LAUNCHES[0] = 0
        blocks = timed(make_step(path, False), args.steps, args.warmup, world, args.repeats)
        launches = native.LAUNCHES[0] // (args.steps * args.repeats + args.warmup)    # per step
        results[path] = dict(block_stats(blocks, args.steps), launches=launches,
                             parity_ok=parity["paths"][path]["ok"],
                             host_enqueue_ms=round(timed.host_ms_per_step, 3))
        if trace.enabled():      # TERRACE_TRACE=events: per-phase device spans, max over ranks
            rep = trace.report(group=True if world > 1 else None)
            if rank == 0:
                print(f"--- phases of path {path} ---\n" + trace.format_report(rep),
                      file=sys.stderr)
    clocks = sampler.stop() if sampler else None
    for path in runners:
        if path.endswith("_pull"):
            continue
        dc = runners[path].time_dispatch_combine(x_dev.detach(), args.steps, args.warmup)
        results[path]["dispatch_combine_us"] = dc
        if world > 1 and dc == dc and dc > 0:      # NVLink roofline of the communication alone
            from terracemoe_simulator_b200.sim import b200_roofline as br
            led = br.egress_bytes(path, TOKENS, TOP_K, TOP_GROUPS, D_MODEL, world, RPN[world])
            results[path]["nvlink_mb_per_direction"] = led["total"] / 1e6
            results[path]["dispatch_combine_frac_of_measured_link"] = \
                2.0 * br.roofline_ms(led["total"]) * 1e3 / dc
    status = native.take_status(local)
    usable = [p for p in runners if results[p]["parity_ok"]] or list(runners)
    best = min(usable, key=lambda p: results[p]["ms_per_step"])
    final = {}
    if trace.enabled():
        trace.report(group=True if world > 1 else None)      # drop the communication-only spans
    e2e_blocks = timed(make_step(best, True), args.steps, args.warmup, world, args.repeats,
                       drain=lambda: final.update(loss=losses.flush()))
    e2e = block_stats(e2e_blocks, args.steps)
    e2e_host_ms = round(timed.host_ms_per_step, 3)
    if trace.enabled():
        rep = trace.report(group=True if world > 1 else None)
        if rank == 0:
            print(f"--- phases of the end-to-end run ({best}) ---\n" + trace.format_report(rep),
                  file=sys.stderr)
    last_loss = final.get("loss")
    tokens = TOKENS * world
    value = tokens / (results[best]["ms_per_step"] * 1e-3)
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
    flops = 3 * 2 * 3 * TOKENS * TOP_K * D_MODEL * D_EXPERT          # fwd + 2x bwd, 3 matrices
    peak_tf = peaks.get("bf16_tflops_sustained", 1400.0)
    ctx0 = runners[best].ctx
    if world == 1:
        transport = "local kernels (no communication)"
    elif args.nccl_arm:
        transport = "nccl all_to_all"
    else:
        transport = "fused peer-memory kernels"
    out = {
        "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": results[best]["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": bench_config(world),
        "impl_detail": {"path": best, "transport": transport,
                        "schedule": ("overlap" if getattr(ctx0, "overlap", False) else
                                     "remote-read" if ctx0 is not None else "local"),
                        "chunks": len(getattr(ctx0, "chunks", [])) or None,
                        "ep_pipeline": int(os.environ.get("TERRACE_EP_PIPELINE", "1") or 1),
                        "timed_blocks": args.repeats,
                        "value_is": "median block of K steps"},
        "paths": results,
        "parity": parity,
        "status": status,
        "gemm_frac_of_measured_sustained": flops / (results[best]["ms_per_step"] * 1e-3) / (peak_tf * 1e12),
        "clocks": clocks,
        "e2e": {"value": tokens / (e2e["ms_per_step"] * 1e-3), "unit": "tokens/s",
                "ms_per_step": e2e["ms_per_step"], "ms_min": e2e["ms_min"], "ms_max": e2e["ms_max"],
                "host_enqueue_ms": e2e_host_ms, "variant": args.e2e_variant,
                "h2d_bytes_per_step": x_host.numel() * 2,
                "d2h_bytes_per_step": losses.bytes_per_read, "last_loss": last_loss},
        "gpu_launches": results[best]["launches"] * args.steps,
    }
    return out


def bench_config(world: int) -> dict:
    """The benchmark configuration, identical for both implementations."""
    return {"model": "single MoE layer d4096 E64x1408 top6 M2", "global_batch": TOKENS * world,
            "seq_len": TOKENS, "parallelism": f"ep{world}",
            "routing_groups": ROUTING_GROUPS[world], "rpn": RPN[world],
            "step": "router+dispatch+experts+combine fwd+bwd",
            "l2": "inputs larger than L2 (expert weights 2.2 GB per step)"}


def run_reference(args, rank, world, local):
    import torch
    import torch.distributed as dist
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "terrace")):
        return {"impl": "reference", "unavailable": "baseline/_ref/terrace is missing"}
    sys.path.insert(0, ref_root)
    from terrace.ep_dist import ep_moe_forward            # noqa: E402  (reference code)
    from terrace.routing import TRouteConfig, t_route     # noqa: E402
    from terrace.ta2a_fwd import init_ta2a_groups, ta2a_moe_forward  # noqa: E402

    device = torch.device("cuda", local)
    router_w, w13, w2, x_host, gy = make_problem(rank, world, device)
    cfg = TRouteConfig(N_EXPERTS, ROUTING_GROUPS[world], TOP_K, TOP_GROUPS)
    params = [t.requires_grad_(True) for t in (router_w, w13, w2)]
    bias = torch.zeros(N_EXPERTS, device=device)
    rpn = RPN[world]
    paths = ["one_hop"]
    if world // rpn >= 2:
        init_ta2a_groups(world, rpn)
        paths.append("two_hop")
    x_dev = x_host.to(device).requires_grad_(True)
    gy_flat, inv_n = gy.reshape(-1), 1.0 / gy.numel()

    def make_step(path, e2e):
        def step():
            for p in params:
                p.grad = None
            if e2e:
                x = x_host.to(device, non_blocking=True).requires_grad_(True)
            else:
                x = x_dev
                x.grad = None
            aff = torch.sigmoid(x @ router_w.t())
            idx, gates, _ = t_route(aff, bias, cfg, "full")
            if path == "one_hop":
                y = ep_moe_forward(x, idx, gates.to(x.dtype), w13, w2, world, N_EXPERTS)
            else:
                y = ta2a_moe_forward(x, idx, gates.to(x.dtype), w13, w2, world, N_EXPERTS,
                                     rpn=rpn, groups_m=TOP_GROUPS)
            if e2e:
                loss = torch.dot(y.reshape(-1).to(gy_flat.dtype), gy_flat) * inv_n   # one reduction
                loss.backward()
                return loss.item()
            y.backward(gy)
            return None
        return step

    results = {}
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    for path in paths:
        blocks = timed(make_step(path, False), args.steps, args.warmup, world, args.repeats)
        results[path] = block_stats(blocks, args.steps)
    clocks = sampler.stop() if sampler else None
    best = min(paths, key=lambda p: results[p]["ms_per_step"])
    e2e = block_stats(timed(make_step(best, True), args.steps, args.warmup, world, args.repeats),
                      args.steps)
    tokens = TOKENS * world
    return {
        "metric": "moe_layer_tokens_per_s",
        "value": tokens / (results[best]["ms_per_step"] * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": results[best]["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": bench_config(world),
        "impl_detail": {"path": best,
                        "transport": "reference torch ops over NCCL all_to_all_single + cuBLAS",
                        "timed_blocks": args.repeats, "value_is": "median block of K steps"},
        "paths": results, "clocks": clocks,
        "e2e": {"value": tokens / (e2e["ms_per_step"] * 1e-3), "unit": "tokens/s",
                "ms_per_step": e2e["ms_per_step"],
                "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": 2},
        "gpu_launches": 0,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--repeats", type=int, default=5,
                    help="timed blocks of K steps each; the median block is reported")
    ap.add_argument("--e2e-variant", default="default",
                    choices=["default", "ungated", "no_h2d", "no_read"],
                    help="diagnosis of the end-to-end number (the reported line says which): "
                         "ungated = start every host-to-device copy at once instead of under the "
                         "weight-gradient GEMMs; no_h2d / no_read = leave out the per-step copy / "
                         "the read-back of the loss")
    ap.add_argument("--no-parity", action="store_true",
                    help="skip the 512-token parity step (for profiler captures)")
    ap.add_argument("--no-ab", action="store_true",
                    help="skip the remote-read schedule that is timed beside the default one")
    ap.add_argument("--nccl-arm", action="store_true",
                    help="ours, but dispatch/combine over NCCL all_to_all instead of fused kernels")
    args = ap.parse_args()
    if args.gpus not in ROUTING_GROUPS:
        raise SystemExit("--gpus must be 1, 2, 4 or 8")
    import torch
    if not torch.cuda.is_available():
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "no CUDA device on this host"}))
            return 0
        raise SystemExit("bench.py needs a CUDA device")
    rank, world, local = setup_dist(args.gpus, force=args.impl == "reference" or args.nccl_arm)
    try:
        out = run_reference(args, rank, world, local) if args.impl == "reference" \
            else run_ours(args, rank, world, local)
    except Exception as exc:  # noqa: BLE001
        if args.impl == "reference":
            out = {"impl": "reference", "unavailable": f"{type(exc).__name__}: {exc}"[:300]}
        else:
            raise
    if rank == 0:
        print(json.dumps(out))
    import torch.distributed as dist
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
