"""Closed-form breakeven bandwidth ratio for the two-hop all-to-all (byte ledger only).

    python -m terracemoe_simulator_b200.tools.breakeven --ratio R [--dies 8] [--epr 4] [--dedup]

Per token and group, two-hop sends ONE row over the slow side instead of q, and adds q rows
(or, with card-level dedup, the expected number D(q) of distinct GPUs hit) on the fast side of
which 1/R stay local:  r_be = (1 - 1/R) * q / (q - 1)   [q -> D(q) with --dedup],
D(q) = R * (1 - C(S-E, q) / C(S, q)), S = R*E experts per group.  Three verdicts: clears with
margin, marginal (< 10 %), or too flat.  Counterpart of the reference's ``tools/breakeven.py``
(:61-130); cross-checked against the full cost model by the tests.
"""
from __future__ import annotations

import argparse
import sys
from math import comb

MARGINAL = 0.10


def D_of(q: int, R: int, E: int) -> float:
    """Expected number of distinct GPUs of a group that q picks among its R*E experts hit."""
    S = R * E
    if q <= 0 or q > S:
        return 0.0
    return R * (1.0 - comb(S - E, q) / comb(S, q))


def breakeven(q: int, R: int, dedup: bool = False, E: int = 4) -> float:
    if q <= 1:
        return float("inf")
    fast_rows = D_of(q, R, E) if dedup else q
    return fast_rows * (1.0 - 1.0 / R) / (q - 1)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Breakeven bandwidth ratio for two-hop all-to-all")
    ap.add_argument("--ratio", type=float, default=None,
                    help="measured fast-side / slow-side bandwidth of your cluster")
    ap.add_argument("--dies", type=int, default=8, help="GPUs (dies) R per group")
    ap.add_argument("--epr", type=int, default=4, help="experts per GPU (only with --dedup)")
    ap.add_argument("--dedup", action="store_true", help="two-hop dedupes at GPU level")
    args = ap.parse_args(argv)
    R = args.dies
    print("Breakeven bandwidth ratio for two-hop all-to-all (R=%d dies per group)" % R)
    print()
    print("  q (experts per group)   r_be%s" % (" (die-level dedup)" if args.dedup else ""))
    rows = []
    for q in range(2, 13):
        r = breakeven(q, R, args.dedup, args.epr)
        rows.append((q, r))
        mark = ""
        if args.ratio is not None:
            mark = "   <- your %.2f is %s" % (args.ratio, "enough" if args.ratio > r else "not enough")
        print("  %2d               %7.4f%s" % (q, r, mark))
    print()
    if args.ratio is None:
        print("Add --ratio <measured ratio> for a verdict.  Use measured values, not nameplate:")
        print("nameplate and effective collective bandwidth often differ by more than 2x.")
        return 0
    good = [(q, r) for q, r in rows if args.ratio > r]
    if not good:
        print("Ratio %.2f does not clear the breakeven line at any quota -- the interconnect is "
              "too flat for this method, do not use two-hop.  The routing constraint of T-Route "
              "can still be evaluated on its own." % args.ratio)
        return 0
    margin = max(args.ratio / r - 1.0 for _, r in good)
    qs = [q for q, _ in good]
    if margin < MARGINAL:
        print("Ratio %.2f only scrapes past the line at q in %s, max margin %.1f%% -- marginal "
              "case, almost certain to be eaten by the fixed-cost side; do not adopt."
              % (args.ratio, qs, margin * 100))
    else:
        print("At ratio %.2f, two-hop comes out ahead on bytes at q in %s (max margin %.0f%%) -- "
              "worth an integration experiment.  Next: audit the fixed cost of the extra "
              "exchange." % (args.ratio, qs, margin * 100))
    return 0


if __name__ == "__main__":
    sys.exit(main())
