"""The one measured two-hop win of the reference: one-hop against Hop A + arrival chain + Hop B +
splits read-back, each timed alone, across a supernode boundary (128 ranks of Ascend 910C, 8 nodes
per supernode, T = 4096 tokens per rank, k = 6).  Two-hop wins all four configurations by 1.43x
to 2.23x; the cost model called all four and misses G by 14 % in the median (9 % once the slow
level is a pure cross-boundary tier).  Communication-call level only.

Parity with the reference ``sim/twohop_measured.py`` (:105-154).  The B200 counterpart with this
repository's own measurements is ``sim/validate_b200.py``.
"""
from __future__ import annotations

from typing import NamedTuple

from .records import TWOHOP_MEASURED as MEASURED

TOKENS, K, N_GROUPS, CARDS_PER_GROUP = 4096, 6, 2, 64
BOUNDARY = "pool110/pool12"
CHAIN_US_PER_ROW_MEASURED = 0.0424
MODEL_ERROR = {"slow level fed a mixture": 0.140, "slow level as a pure tier": 0.090,
               "pure tier and measured chain": 0.151}
PURE_CROSS_BOUNDARY_GBPS = 7.9


class Run(NamedTuple):
    """One measured configuration: the one-hop call and the four parts of the two-hop call, ms."""
    H: int
    M: int
    q: int
    one_hop: float
    hop_a: float
    chain: float
    hop_b: float
    splits: float

    @property
    def two_hop(self) -> float:
        return sum(self[4:])

    @property
    def gain(self) -> float:
        return self.one_hop / self.two_hop


def two_hop_ms(row) -> float:
    return Run(*row).two_hop


def g(row) -> float:
    return Run(*row).gain


def chain_share(row) -> float:
    run = Run(*row)
    return run.chain / run.two_hop


def every_configuration_wins() -> bool:
    return min(map(g, MEASURED)) > 1.0


def main() -> None:
    from ._text import Column, render_table
    runs = [Run(*row) for row in MEASURED]
    print("One hop against two, measured across the %s supernode boundary." % BOUNDARY)
    print("128 ranks, 8 nodes in each supernode, T = %d tokens per rank, k = %d.\n" % (TOKENS, K))
    cols = [Column(name, "%-" + str(width) + "d", lambda r, i=i: r[i])
            for i, (name, width) in enumerate((("H", 6), ("M", 4), ("q", 4)))]
    cols += [Column(name, fmt, lambda r, i=i: r[i]) for i, name, fmt in
             ((3, "one hop", "%9.3f"), (4, "hop A", "%8.3f"), (5, "chain", "%8.3f"),
              (6, "hop B", "%8.3f"), (7, "splits", "%8.3f"))]
    cols += [Column("two hop", "%9.3f", lambda r: r.two_hop), Column("G", "%7.3f", lambda r: r.gain),
             Column("", "%-4s", lambda r: "WIN" if r.gain > 1.0 else "loss")]
    print("\n".join(render_table(cols, runs)))
    gains = sorted(r.gain for r in runs)
    print("\nTwo-hop wins in %d of %d configurations, by %.2fx to %.2fx."
          % (sum(x > 1.0 for x in gains), len(gains), gains[0], gains[-1]))
    print("Model error on G: %.0f%% median with the slow level fed a mixture, %.0f%% as a pure "
          "%.1f GB/s tier." % (100 * MODEL_ERROR["slow level fed a mixture"],
                              100 * MODEL_ERROR["slow level as a pure tier"],
                              PURE_CROSS_BOUNDARY_GBPS))
    print("Arrival chain: %.4f us per pair measured in situ." % CHAIN_US_PER_ROW_MEASURED)
    print("Communication-call level only; nothing here is a claim about training throughput.")


if __name__ == "__main__":
    main()
