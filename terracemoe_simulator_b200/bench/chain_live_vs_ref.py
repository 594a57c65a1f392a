"""The arrival step as the closed forward runs it against its specification, one shape.

``chain_sweep`` covers the grid; this is the single-shape check the reference keeps beside it
(``bench/chain_live_vs_ref.py:29-72``): the shapes of one two-hop dispatch (T*M received rows,
quota q) timed through ``ops.k1_arrival`` and through ``k1_arrival_ref``, plus a bitwise
comparison of the two results, so that a timing is never quoted for a path that computes
something else.

    python -m terracemoe_simulator_b200.bench.chain_live_vs_ref [--tokens 4096 --hidden 2048]
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from .chain_sweep import time_ms


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--k", type=int, default=6)
    ap.add_argument("--m", type=int, default=2)
    ap.add_argument("--epr", type=int, default=4)
    ap.add_argument("--rpn", type=int, default=8)
    ap.add_argument("--calls", type=int, default=9)
    ap.add_argument("--cpu", action="store_true")
    args = ap.parse_args(argv)
    from .. import ops
    from ..ops.refs import k1_arrival_ref
    device = torch.device("cuda" if torch.cuda.is_available() and not args.cpu else "cpu")
    q, n_rows = args.k // args.m, args.tokens * args.m
    g = torch.Generator().manual_seed(0)
    rx = torch.randn(n_rows, args.hidden, generator=g).to(torch.bfloat16).to(device)
    rslot = torch.randint(0, args.rpn * args.epr, (n_rows, q), generator=g).sort(dim=1).values
    rslot = rslot.to(device)
    rgate = torch.rand(n_rows, q, generator=g).to(torch.bfloat16).to(device)
    live = ops.k1_arrival(rx, rslot, rgate, quota=q, epr=args.epr, rpn=args.rpn)
    ref = k1_arrival_ref(rx, rslot, rgate, q, args.epr, args.rpn)
    same = all(torch.equal(a, b) for a, b in zip(live, ref))
    out = {"device": str(device), "native": bool(ops.custom_ops_enabled()), "rows": n_rows,
           "pairs": n_rows * q, "hidden": args.hidden, "bitwise_equal": same,
           "live_ms": time_ms(lambda: ops.k1_arrival(rx, rslot, rgate, quota=q, epr=args.epr,
                                                     rpn=args.rpn), args.calls, device),
           "ref_ms": time_ms(lambda: k1_arrival_ref(rx, rslot, rgate, q, args.epr, args.rpn),
                             args.calls, device)}
    out["live_over_ref"] = out["live_ms"] / max(out["ref_ms"], 1e-12)
    print(json.dumps(out))
    return 0 if same else 1


if __name__ == "__main__":
    sys.exit(main())
