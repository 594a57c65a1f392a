"""Does the fixed cost of an all-to-all add to its transfer time, or overlap it?

The cost model prices a call as ``alpha(world) + bytes / beta``.  The alternative, the two
terms overlapping (combining in quadrature), cannot be told apart at tiny sizes (both give
alpha) or huge ones (both give bytes / beta); they differ most where the two terms are equal,
so the size grid is dense through that decade.  Both timing styles run at the same world over
the same sizes, so a difference between them is the instrument, not the machine.

    python -m torch.distributed.run --nproc-per-node N \
        -m terracemoe_simulator_b200.bench.a2a_form_probe --out a2a_form.json

The JSON rows carry ``{world, bytes, per_peer_bytes, burst_ms, percall_ms, *_spread}`` and
``records`` in the fitting schema ``{frame, world, bytes, ms}`` (frames ``burst`` / ``percall``)
that ``sim.fit`` and ``sim.hostregime`` read.  Counterpart of the reference's
``bench/a2a_form_probe.py:47-134``; on NVSwitch alpha is a few tens of microseconds and beta
several hundred GB/s, so the crossing sits near 16-32 MB instead of 13 MB.
"""
from __future__ import annotations

import argparse
import sys

import torch
import torch.distributed as dist

from . import harness as hz

SIZES_MIB = [0.0625, 0.125, 0.25, 0.5, 1, 1.5, 2, 3, 4, 6, 8, 10, 12, 16, 20, 24, 32, 48, 64,
             96, 128, 192, 256]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--out", required=True)
    ap.add_argument("--sizes-mib", type=float, nargs="+", default=SIZES_MIB)
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--burst-n", type=int, default=32)
    ap.add_argument("--percall-n", type=int, default=11)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--tag", default="")
    args = ap.parse_args(argv)
    env = hz.init(args.cpu)
    rows, records = [], []
    for mib in args.sizes_mib:
        nbytes = int(mib * 1024 * 1024)
        if nbytes % (env.world * 32):           # per-peer slices stay 16-byte aligned
            continue
        inp = torch.ones(nbytes // 2, dtype=torch.bfloat16, device=env.device)
        out = torch.empty_like(inp)
        call = lambda: dist.all_to_all_single(out, inp)   # noqa: E731
        for _ in range(args.warmup):
            call()
        hz.sync(env)
        b, bs = hz.median_of(env, hz.burst, call, args.burst_n, args.repeats)
        p, ps = hz.median_of(env, hz.percall, call, args.percall_n, args.repeats)
        rows.append({"world": env.world, "bytes": nbytes, "per_peer_bytes": nbytes / env.world,
                     "burst_ms": b, "burst_spread": bs, "percall_ms": p, "percall_spread": ps})
        records += [{"frame": "burst", "world": env.world, "bytes": nbytes, "ms": b},
                    {"frame": "percall", "world": env.world, "bytes": nbytes, "ms": p}]
        hz.say(env, "%10d B  per-peer %9.0f B   burst %8.4f ms (spread %4.1f%%)   percall %8.4f ms "
                    "(spread %4.1f%%)   ratio %.2f" % (nbytes, nbytes / env.world, b, 100 * bs, p,
                                                       100 * ps, p / max(b, 1e-12)))
        del inp, out
    hz.write_json(env, args.out, {"tag": args.tag, "world": env.world, "burst_n": args.burst_n,
                                  "percall_n": args.percall_n, "repeats": args.repeats,
                                  "rows": rows, "records": records})
    hz.finish(env)
    return 0


if __name__ == "__main__":
    sys.exit(main())
