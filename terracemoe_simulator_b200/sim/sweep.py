"""Communication-level extrapolation table: one-hop/two-hop time ratio against the hierarchy
ratio of a synthetic cluster, for three implementation tiers of the arrival chain.  Refuses to
print anything when the Tier-1 gate fails; reports (but does not require) the Tier-2 gate.

Parity with the reference ``sim/sweep.py`` (``CHAIN_SCENARIOS`` :22-28, ``comm_speedup`` :31-37,
``main`` :40-75).
"""
from __future__ import annotations

from . import calibrate as cal
from ._text import Column, render_table

CHAIN_SCENARIOS = [
    ("PyTorch chain (measured)", cal.CHAIN_US_PER_ROW),
    ("hypothetical fused target", 0.012),
    ("zero implementation overhead (upper bound)", 0.0),
]
RATIOS = (1.03, 2.0, 3.2, 4.5, 8.0, 15.7)
READING = """How to read:
  - The flat column (1.03) stays <=1 at every tier: on a machine without hierarchy
    the two-hop exchange does not pay for its extra hop.
  - Columns with ratio >= 3.2 are all >1; the ratios are synthetic scenarios, not
    target measurements, and the tier changes the magnitude materially."""


def comm_speedup(cluster, q: int, tok: int, k_base: int = 6) -> float:
    """one-hop / two-hop dispatch time on 16 groups of ``cluster.R`` ranks with quota ``q``."""
    from .uncertainty import Shape
    return Shape.for_quota(q, tok, cluster.R, k_base).speedup(cluster)


def ratio_table(qs=(2, 3, 6), tok: int = 4096) -> dict:
    """{tier name: {q: [speedup at every ratio of RATIOS]}}"""
    table = {}
    for tier, chain in CHAIN_SCENARIOS:
        family = [cal.synthetic(ratio, chain_us_per_row=chain) for ratio in RATIOS]
        table[tier] = {q: [comm_speedup(c, q, tok) for c in family] for q in qs}
    return table


def _gates(cluster) -> tuple:
    from .validate import validate
    from .validate_micro import validate_micro
    return validate_micro(cluster, verbose=False)[0], validate(cluster, verbose=False)[0]


def main() -> None:
    micro_ok, step_ok = _gates(cal.aug_flat())
    print("Tier-1 (communication level): %s" % ("PASS" if micro_ok else "FAIL"))
    print("Tier-2 (step level): %s" % ("PASS" if step_ok
                                       else "FAIL -- step-level extrapolation locked"))
    if not micro_ok:
        raise SystemExit("Tier-1 fails; all extrapolation forbidden.")
    bar = "=" * 74
    print("\n%s\nCommunication-level extrapolation (simulation, not measurement)" % bar)
    print("x-axis = fast/slow bandwidth ratio; cell = one-hop time / two-hop time "
          "(>1 = two-hop faster)")
    print("Geometry: 16 groups x R=8, k=6, T=4096 tok/rank\n%s" % bar)
    columns = [Column("q \\ ratio", "%-16s", lambda item: "q=%d" % item[0])]
    columns += [Column("ratio %g" % r, "%12.2f", lambda item, i=i: item[1][i])
                for i, r in enumerate(RATIOS)]
    for (tier, chain), cells in zip(CHAIN_SCENARIOS, ratio_table().values()):
        print("\n-- implementation tier: %s (%.4f us/row) --" % (tier, chain))
        print("\n".join(render_table(columns, cells.items())))
    print("\n" + READING)


if __name__ == "__main__":
    main()
