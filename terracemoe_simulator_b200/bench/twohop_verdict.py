"""One collective against the two-hop phases, each timed alone, at real dispatch shapes.

For hidden width H in {2048, 4096} and M in {1, 2} (k = 6, 4096 tokens per rank) it times

* ``one_hop``  one all-to-all of T*k rows over every rank,
* ``hop_a``    T*M rows to the group representatives (one peer per group, this rank's own
  group served by a local copy),
* ``chain``    the arrival step on the received rows (``ops.k1_arrival``: the sm_100a kernel
  when the native library is loaded, its PyTorch specification otherwise),
* ``hop_b``    T*k rows inside the group,
* ``splits``   the device-to-host readback a variable-length collective cannot avoid,

percall style, MAX over ranks, and reports ``G = one_hop / (hop_a + chain + hop_b + splits)``.
The ranks are split into ``world / rpn`` groups of ``--rpn`` ranks.  This is the measurement
``sim/twohop_measured.py`` records for the reference machine (``bench/twohop_verdict.py:50-166``
there); the fused kernels of this package remove ``chain`` and ``splits`` altogether, which
``bench.py`` measures.

    python -m torch.distributed.run --nproc-per-node 8 \
        -m terracemoe_simulator_b200.bench.twohop_verdict --rpn 2 --out verdict.json
"""
from __future__ import annotations

import argparse
import sys

import torch
import torch.distributed as dist

from . import harness as hz


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--out", required=True)
    ap.add_argument("--rpn", type=int, default=2, help="ranks per group")
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--k", type=int, default=6)
    ap.add_argument("--hidden", type=int, nargs="+", default=[2048, 4096])
    ap.add_argument("--epr", type=int, default=4, help="experts per rank")
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--calls", type=int, default=7)
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--tag", default="")
    args = ap.parse_args(argv)
    env = hz.init(args.cpu)
    from .. import ops
    world, rpn = env.world, args.rpn
    if world % rpn or world // rpn < 2:
        raise SystemExit("need at least two groups of --rpn ranks")
    n_groups = world // rpn
    groups = [dist.new_group(ranks=list(range(g * rpn, (g + 1) * rpn))) for g in range(n_groups)]
    mine = groups[env.rank // rpn]
    reps = [g * rpn + env.rank % rpn for g in range(n_groups)]     # Hop A peers of this rank
    T, K = args.tokens, args.k
    rows = []
    for H in args.hidden:
        for M in (1, 2):
            if K % M or M > n_groups:
                continue
            q = K // M
            one = torch.ones(T * K // world * world, H, dtype=torch.bfloat16, device=env.device)
            one_out = torch.empty_like(one)
            per = T * M // n_groups
            split = [per if r in reps else 0 for r in range(world)]
            a_in = torch.ones(per * n_groups, H, dtype=torch.bfloat16, device=env.device)
            a_out = torch.empty_like(a_in)
            rx = torch.randn(T * M, H, device=env.device).to(torch.bfloat16)
            rslot = torch.randint(0, rpn * args.epr, (T * M, q),
                                  device=env.device).sort(dim=1).values
            rgate = torch.randn(T * M, q, device=env.device).to(torch.bfloat16)
            b_in = torch.ones(T * K // rpn * rpn, H, dtype=torch.bfloat16, device=env.device)
            b_out = torch.empty_like(b_in)
            cnt = torch.zeros(rpn, dtype=torch.int32, device=env.device)
            phases = {
                "one_hop": lambda: dist.all_to_all_single(one_out, one),
                "hop_a": lambda: dist.all_to_all_single(a_out, a_in, split, split),
                "chain": lambda: ops.k1_arrival(rx, rslot, rgate, quota=q, epr=args.epr, rpn=rpn),
                "hop_b": lambda: dist.all_to_all_single(b_out, b_in, group=mine),
                "splits": lambda: cnt.cpu(),
            }
            for name, fn in phases.items():
                for _ in range(3):
                    fn()
            hz.sync(env)
            t = {name: hz.median_of(env, hz.percall, fn, args.calls, args.repeats)[0]
                 for name, fn in phases.items()}
            two = t["hop_a"] + t["chain"] + t["hop_b"] + t["splits"]
            row = {"H": H, "M": M, "q": q, "tokens": T, "k": K, "world": world, "rpn": rpn,
                   "native_chain": bool(ops.custom_ops_enabled()),
                   **{f"{name}_ms": v for name, v in t.items()}, "two_hop_ms": two,
                   "G": t["one_hop"] / max(two, 1e-12)}
            rows.append(row)
            hz.say(env, "H=%5d M=%d q=%d | one-hop %7.3f | hopA %6.3f chain %6.3f hopB %6.3f "
                        "splits %5.3f = two-hop %7.3f | G = %.3f  %s"
                   % (H, M, q, t["one_hop"], t["hop_a"], t["chain"], t["hop_b"], t["splits"], two,
                      row["G"], "TWO-HOP WINS" if row["G"] > 1 else "two-hop loses"))
    hz.write_json(env, args.out, {"tag": args.tag, "world": world, "rows": rows})
    hz.finish(env)
    return 0


if __name__ == "__main__":
    sys.exit(main())
