"""Dispatch/combine sweep for cost-model calibration (run under ``torch.distributed.run``).

    python -m torch.distributed.run --nproc-per-node N -m terracemoe_simulator_b200.bench.sweep \
        --out sweep_N.json [--tokens 256 1024 4096 16384] [--hidden 4096]

For every tokens-per-GPU value, group size R in {2, 4} (where N allows at least two groups) and
quota q in {1, 2, 3, 4} (64 experts, M = 2, k = q*M) it times the fused one-hop and two-hop
dispatch+combine (rows echo back through the owners' buffers; no expert compute), device-timed
with CUDA events, max over ranks, burst style (``--iters`` back-to-back calls, one sync).
It also times the NCCL ``all_to_all_single`` of the same payload as the library baseline.
Output: JSON with ``rows`` (one dict per configuration: both times, bus GB/s, measured
two-hop/one-hop ratio) and ``records`` in the ``sim.fit`` schema ``{frame, world, bytes, ms}``.
Three frames are measured, each as half of a one-hop dispatch + combine of the fused transport:

  ``flat``   all N ranks, T*k rows per rank (the one-hop exchange itself)
  ``slow``   Hop A shaped: the N_g ranks that share a local index (one per group), T*M rows per
             rank, every such peer set exchanging at the same time
  ``fast``   Hop B shaped: the R ranks of a group, T*k rows per rank, all groups at the same time

``slow`` and ``fast`` run on arenas that span only their peer set, so their fixed cost and
bandwidth are the levels' own (``sim.calibrate.b200_from_records`` fits one alpha and one beta
per frame with ``sim.fit.fit_beta_pinned``).  Counterpart of the reference's
``bench/a2a_form_probe.py`` / ``bench/twohop_verdict.py`` measurement protocol (barrier, sync,
timed burst, MAX over ranks).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def _timed(fn, iters, warmup, world, bursts: int = 3):
    """Median over ``bursts`` timed bursts of ``iters`` back-to-back calls each (one burst of a
    50 us call is too noisy to calibrate a fixed cost from); every burst is bracketed by a
    barrier + synchronize and reduced with MAX over ranks."""
    for _ in range(warmup):
        fn()
    seen = []
    for _ in range(bursts):
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        seen.append(ms.item())
    return sorted(seen)[len(seen) // 2]


def _peer_sets(world: int, R: int):
    """(slow sets, fast sets): ranks sharing a local index, and the ranks of each group."""
    groups = world // R
    slow = [[g * R + j for g in range(groups)] for j in range(R)]
    fast = [[g * R + j for j in range(R)] for g in range(groups)]
    return slow, fast


def _level_frames(world, rank, R, T, H, iters, warmup, dev, groups_cache):
    """Half the dispatch + combine time of a one-hop exchange inside this rank's ``slow`` and
    ``fast`` peer sets, with T*M and T*k rows: ``[(frame, peers, bytes, ms)]``."""
    from terracemoe_simulator_b200.parallel import fused as fz
    from terracemoe_simulator_b200.routing import TRouteConfig, t_route
    out = []
    slow_sets, fast_sets = _peer_sets(world, R)
    for frame, sets, k in (("slow", slow_sets, 2), ("fast", fast_sets, 6)):
        n = len(sets[0])
        if n < 2:
            continue
        mine = None
        for members in sets:                      # every rank creates every group, same order
            key = tuple(members)
            if key not in groups_cache:
                groups_cache[key] = dist.new_group(members)
            if rank in members:
                mine = (members, groups_cache[key])
        members, group = mine
        E = 16 * n                                # 16 experts per peer, one routing group
        cfg = TRouteConfig(E, 1, k, 1)
        ctx = fz.FusedEPContext(cfg, H, 64, T, world=n, rank=members.index(rank), rpn=n,
                                device=dev, group=group, row_capacity_factor=3.0)
        g = torch.Generator().manual_seed(77 * rank + T + k)
        x = torch.randn(T, H, generator=g).bfloat16().to(dev)
        idx, gates, _ = t_route(torch.rand(T, E, generator=g).to(dev), torch.zeros(E, device=dev),
                                cfg)
        ms = _timed(lambda: fz.fused_dispatch_combine(ctx, x, idx, gates, mode="one_hop"),
                    iters, warmup, world)
        status = ctx.take_status()
        out.append((frame, n, T * k * H * 2, ms / 2, status))
        ctx.close()
        del ctx
        torch.cuda.empty_cache()
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="sweep.json")
    ap.add_argument("--tokens", type=int, nargs="+", default=[256, 1024, 4096, 16384])
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", local))
    from terracemoe_simulator_b200.parallel import fused as fz
    from terracemoe_simulator_b200.routing import TRouteConfig, t_route
    dev = torch.device("cuda", local)
    H, E, M = args.hidden, args.experts, 2
    rows, records = [], []
    groups_cache: dict = {}
    for R in (2, 4):              # per-level frames: the peer sets of groups of R
        if world % R or world // R < 1:
            continue
        for T in args.tokens:
            for frame, n, nbytes, ms, status in _level_frames(world, rank, R, T, H, args.iters,
                                                              args.warmup, dev, groups_cache):
                rec = {"frame": frame, "world": n, "bytes": nbytes, "ms": ms, "R": R,
                       "tokens": T, "status": status}
                records.append(rec)
                if rank == 0:
                    print(json.dumps(rec), flush=True)
    for R in (1, 2, 4):
        n_nodes = world // R
        if world % R or n_nodes < 2 or E % n_nodes:
            continue
        for q in (1, 2, 3, 4):
            k = q * M
            if M > n_nodes or q > E // n_nodes:
                continue
            cfg = TRouteConfig(E, n_nodes, k, M)
            for T in args.tokens:
                ctx = fz.FusedEPContext(cfg, H, 64, T, world=world, rank=rank, rpn=R, device=dev,
                                        row_capacity_factor=3.0)
                g = torch.Generator().manual_seed(1000 * rank + T + q)
                x = torch.randn(T, H, generator=g).bfloat16().to(dev)
                aff = torch.rand(T, E, generator=g).to(dev)
                idx, gates, _ = t_route(aff, torch.zeros(E, device=dev), cfg)
                res = {}
                for mode in ("one_hop", "two_hop"):
                    res[mode] = _timed(lambda: fz.fused_dispatch_combine(ctx, x, idx, gates,
                                                                         mode=mode),
                                       args.iters, args.warmup, world)
                # NCCL all_to_all of the one-hop payload (both directions), uniform splits
                per = T * k // world
                send = torch.empty(per * world, H, dtype=torch.bfloat16, device=dev)
                recv = torch.empty_like(send)

                def nccl():
                    dist.all_to_all_single(recv, send)
                    dist.all_to_all_single(send, recv)
                res["nccl_a2a_x2"] = _timed(nccl, args.iters, args.warmup, world)
                status = ctx.take_status()
                one_bytes = T * k * H * 2
                row = {"world": world, "R": R, "n_groups": n_nodes, "q": q, "k": k, "M": M,
                       "tokens": T, "hidden": H, "one_hop_ms": res["one_hop"],
                       "two_hop_ms": res["two_hop"], "nccl_a2a_x2_ms": res["nccl_a2a_x2"],
                       "ratio_two_over_one": res["two_hop"] / res["one_hop"],
                       "one_hop_bus_gbs": 2 * one_bytes * (world - 1) / world
                       / (res["one_hop"] * 1e-3) / 1e9,
                       "status": status}
                rows.append(row)
                # dispatch + combine move the payload twice: record half the time per direction
                records.append({"frame": "flat", "world": world, "bytes": one_bytes,
                                "ms": res["one_hop"] / 2})
                ctx.close()
                del ctx
                torch.cuda.empty_cache()
                if rank == 0:
                    print(json.dumps(row), flush=True)
    if rank == 0:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "w") as f:
            json.dump({"rows": rows, "records": records}, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
