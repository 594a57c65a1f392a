"""Closed-form breakeven bandwidth ratio for the two-hop all-to-all (byte ledger only).

    python -m terracemoe_simulator_b200.tools.breakeven --ratio R [--dies 8] [--epr 4] [--dedup]

The ledger, per token and routing group: one-hop sends the token's q rows over the slow side;
two-hop sends ONE row over the slow side and then pays, on the fast side, either q rows or, when
the group forwards one copy per GPU rather than per expert (``--dedup``), the expected number
D(q) of distinct GPUs its q experts sit on; of those fast-side rows 1/R stay on the GPU that
received the slow-side row.  Two-hop wins on bytes when the q - 1 slow-side rows it saves, priced
at the slow rate, outweigh its fast-side rows:

    ratio > r_be = fast_rows * (1 - 1/R) / (q - 1),     D(q) = R * (1 - C(S-E, q) / C(S, q)),

S = R * E experts per group, E per GPU.  The CLI tabulates r_be for q = 2 .. 12 and, given a
measured ratio, says which of three cases applies: clears with margin, marginal (< 10 %), or too
flat.  Counterpart of the reference's ``tools/breakeven.py`` (:61-130); cross-checked against the
full cost model by the tests.
"""
from __future__ import annotations

import argparse
import sys
from dataclasses import dataclass
from math import comb

MARGINAL = 0.10
QUOTAS = range(2, 13)


@dataclass(frozen=True)
class GroupLedger:
    """Rows one token moves for one of its routing groups (R GPUs of E experts each)."""
    q: int
    R: int
    E: int = 4
    dedup: bool = False

    @property
    def distinct_gpus(self) -> float:
        experts = self.R * self.E
        if not 0 < self.q <= experts:
            return 0.0
        miss_one_gpu = comb(experts - self.E, self.q) / comb(experts, self.q)
        return self.R * (1.0 - miss_one_gpu)

    @property
    def fast_rows(self) -> float:
        forwarded = self.distinct_gpus if self.dedup else float(self.q)
        return forwarded * (self.R - 1) / self.R

    @property
    def slow_rows_saved(self) -> int:
        return self.q - 1

    @property
    def breakeven(self) -> float:
        return self.fast_rows / self.slow_rows_saved if self.slow_rows_saved > 0 else float("inf")


def D_of(q: int, R: int, E: int) -> float:
    """Expected number of distinct GPUs of a group that q picks among its R*E experts hit."""
    return GroupLedger(q, R, E).distinct_gpus


def breakeven(q: int, R: int, dedup: bool = False, E: int = 4) -> float:
    return GroupLedger(q, R, E, dedup).breakeven


def verdict(ratio: float, lines: dict) -> str:
    """One of the three verdict sentences for a measured ``ratio`` against ``{q: r_be}``."""
    ahead = {q: ratio / r - 1.0 for q, r in lines.items() if ratio > r}
    if not ahead:
        return ("Ratio %.2f does not clear the breakeven line at any quota -- the interconnect is "
                "too flat for this method, do not use two-hop.  The routing constraint of T-Route "
                "can still be evaluated on its own." % ratio)
    best = max(ahead.values())
    if best < MARGINAL:
        return ("Ratio %.2f only scrapes past the line at q in %s, max margin %.1f%% -- marginal "
                "case, almost certain to be eaten by the fixed-cost side; do not adopt."
                % (ratio, sorted(ahead), 100 * best))
    return ("At ratio %.2f, two-hop comes out ahead on bytes at q in %s (max margin %.0f%%) -- "
            "worth an integration experiment.  Next: audit the fixed cost of the extra exchange."
            % (ratio, sorted(ahead), 100 * best))


def _parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="Breakeven bandwidth ratio for two-hop all-to-all")
    ap.add_argument("--ratio", type=float, default=None,
                    help="measured fast-side / slow-side bandwidth of your cluster")
    ap.add_argument("--dies", type=int, default=8, help="GPUs (dies) R per group")
    ap.add_argument("--epr", type=int, default=4, help="experts per GPU (only with --dedup)")
    ap.add_argument("--dedup", action="store_true", help="two-hop dedupes at GPU level")
    return ap


def main(argv=None) -> int:
    args = _parser().parse_args(argv)
    lines = {q: breakeven(q, args.dies, args.dedup, args.epr) for q in QUOTAS}
    out = ["Breakeven bandwidth ratio for two-hop all-to-all (R=%d dies per group)" % args.dies,
           "", "  q (experts per group)   r_be" + (" (die-level dedup)" if args.dedup else "")]
    for q, r in lines.items():
        note = ""
        if args.ratio is not None:
            note = "   <- your %.2f is %senough" % (args.ratio, "" if args.ratio > r else "not ")
        out.append("  %2d               %7.4f%s" % (q, r, note))
    out.append("")
    if args.ratio is None:
        out += ["Add --ratio <measured ratio> for a verdict.  Use measured values, not nameplate:",
                "nameplate and effective collective bandwidth often differ by more than 2x."]
    else:
        out.append(verdict(args.ratio, lines))
    print("\n".join(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
