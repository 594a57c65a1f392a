"""Does per-pair bandwidth hold when many GPU pairs cross the switch at once?

Structure is held fixed and only pressure varies: the ranks are split into two halves, rank i
pairs with rank i + world/2, and each pair runs the same two-rank all-to-all while 1, 2, 4 ...
pairs are active concurrently (idle pairs wait at the next barrier).  Every active pair does
identical work at every step, so a slowdown is contention in the fabric and nothing else.  A
last phase times one all-to-all over every rank, the pattern expert parallelism really uses.
Percall style (ranks aligned, one call timed, MAX over the active ranks).

On an NVSwitch domain every pair has a dedicated 900 GB/s path, so the expected result is a flat
line; the reference ran the same design across a supernode boundary, where uplinks are shared
(``bench/xsupernode_contention.py:57-142``), and a flat line there is what lets the cost model
price cross-boundary bytes without a contention term.

    python -m torch.distributed.run --nproc-per-node 8 \
        -m terracemoe_simulator_b200.bench.fabric_contention --out contention.json
"""
from __future__ import annotations

import argparse
import sys

import torch
import torch.distributed as dist

from . import harness as hz

SIZES_MIB = [32, 64, 128]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--out", required=True)
    ap.add_argument("--sizes-mib", type=float, nargs="+", default=SIZES_MIB)
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--calls", type=int, default=7)
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--tag", default="")
    args = ap.parse_args(argv)
    env = hz.init(args.cpu)
    if env.world < 2 or env.world % 2:
        raise SystemExit("needs an even number of ranks")
    half = env.world // 2
    my_pair = env.rank % half
    groups = [dist.new_group(ranks=[p, p + half]) for p in range(half)]   # same order everywhere
    mine = groups[my_pair]
    levels = [n for n in (1, 2, 4, 8, 16) if n <= half]
    rows = []
    for mib in args.sizes_mib:
        nbytes = int(mib * 1024 * 1024)
        inp = torch.ones(nbytes // 2, dtype=torch.bfloat16, device=env.device)
        out = torch.empty_like(inp)
        call = lambda: dist.all_to_all_single(out, inp, group=mine)     # noqa: E731
        for _ in range(3):
            call()
        hz.sync(env)
        for active in levels:
            on = my_pair < active
            work = call if on else (lambda: None)
            ts = []
            for _ in range(args.repeats):
                t = hz.percall(env, work, args.calls)       # MAX over every rank: idle ranks add 0
                ts.append(t)
            ts.sort()
            ms = ts[len(ts) // 2]
            rows.append({"phase": "pairs", "active_pairs": active, "bytes": nbytes, "ms": ms,
                         "spread": hz.spread(ts), "gbs_per_rank": nbytes / 2 / (ms * 1e-3) / 1e9})
            hz.say(env, "  %6.1f MiB  %2d active pair(s)  %8.4f ms  %7.1f GB/s per rank and direction"
                   % (mib, active, ms, rows[-1]["gbs_per_rank"]))
        if (nbytes // 2) % env.world == 0:
            gout = torch.empty_like(inp)
            gcall = lambda: dist.all_to_all_single(gout, inp)           # noqa: E731
            for _ in range(3):
                gcall()
            ms, sp = hz.median_of(env, hz.percall, gcall, args.calls, args.repeats)
            rows.append({"phase": "global", "active_pairs": half, "bytes": nbytes, "ms": ms,
                         "spread": sp, "gbs_per_rank": nbytes * (env.world - 1) / env.world
                         / (ms * 1e-3) / 1e9})
            hz.say(env, "  %6.1f MiB  all-to-all over %d ranks  %8.4f ms" % (mib, env.world, ms))
            del gout
        del inp, out
    base = {r["bytes"]: r["ms"] for r in rows if r["phase"] == "pairs" and r["active_pairs"] == 1}
    worst = max((r["ms"] / base[r["bytes"]] for r in rows if r["phase"] == "pairs"), default=1.0)
    hz.say(env, "worst slowdown against one active pair: %.2fx" % worst)
    hz.write_json(env, args.out, {"tag": args.tag, "world": env.world, "rows": rows,
                                  "worst_slowdown": worst})
    hz.finish(env)
    return 0


if __name__ == "__main__":
    sys.exit(main())
