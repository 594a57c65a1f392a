"""The one measured two-hop win of the reference: one-hop against Hop A + arrival chain + Hop B +
splits read-back, each timed alone, across a supernode boundary (128 ranks of Ascend 910C, 8 nodes
per supernode, T = 4096 tokens per rank, k = 6).  Two-hop wins all four configurations by 1.43x
to 2.23x; the cost model called all four and misses G by 14 % in the median (9 % once the slow
level is a pure cross-boundary tier).  Communication-call level only.

Parity with the reference ``sim/twohop_measured.py`` (:105-154).  The B200 counterpart with this
repository's own measurements is ``sim/validate_b200.py``.
"""
from __future__ import annotations

from .records import TWOHOP_MEASURED as MEASURED

TOKENS, K, N_GROUPS, CARDS_PER_GROUP = 4096, 6, 2, 64
BOUNDARY = "pool110/pool12"
CHAIN_US_PER_ROW_MEASURED = 0.0424
MODEL_ERROR = {"slow level fed a mixture": 0.140, "slow level as a pure tier": 0.090,
               "pure tier and measured chain": 0.151}
PURE_CROSS_BOUNDARY_GBPS = 7.9


def two_hop_ms(row) -> float:
    return row[4] + row[5] + row[6] + row[7]


def g(row) -> float:
    return row[3] / two_hop_ms(row)


def every_configuration_wins() -> bool:
    return all(g(r) > 1.0 for r in MEASURED)


def chain_share(row) -> float:
    return row[5] / two_hop_ms(row)


def main() -> None:
    print("One hop against two, measured across the %s supernode boundary." % BOUNDARY)
    print("128 ranks, 8 nodes in each supernode, T = %d tokens per rank, k = %d." % (TOKENS, K))
    print()
    print("%-6s %-4s %-4s %9s %8s %8s %8s %8s %9s %7s" % ("H", "M", "q", "one hop", "hop A",
                                                          "chain", "hop B", "splits", "two hop",
                                                          "G"))
    for r in MEASURED:
        print("%-6d %-4d %-4d %9.3f %8.3f %8.3f %8.3f %8.3f %9.3f %7.3f %s"
              % (r + (two_hop_ms(r), g(r), "WIN" if g(r) > 1 else "loss")))
    gs = [g(r) for r in MEASURED]
    print()
    print("Two-hop wins in %d of %d configurations, by %.2fx to %.2fx."
          % (sum(x > 1 for x in gs), len(gs), min(gs), max(gs)))
    print("Model error on G: %.0f%% median with the slow level fed a mixture, %.0f%% as a pure "
          "%.1f GB/s tier." % (100 * MODEL_ERROR["slow level fed a mixture"],
                              100 * MODEL_ERROR["slow level as a pure tier"],
                              PURE_CROSS_BOUNDARY_GBPS))
    print("Arrival chain: %.4f us per pair measured in situ." % CHAIN_US_PER_ROW_MEASURED)
    print("Communication-call level only; nothing here is a claim about training throughput.")


if __name__ == "__main__":
    main()
