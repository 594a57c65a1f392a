"""Communication-level extrapolation table: one-hop/two-hop time ratio against the hierarchy
ratio of a synthetic cluster, for three implementation tiers of the arrival chain.  Refuses to
print anything when the Tier-1 gate fails; reports (but does not require) the Tier-2 gate.

Parity with the reference ``sim/sweep.py`` (``CHAIN_SCENARIOS`` :22-28, ``comm_speedup`` :31-37,
``main`` :40-75).
"""
from __future__ import annotations

from .calibrate import CHAIN_US_PER_ROW, aug_flat, synthetic
from .core import MoEGeometry, one_hop_call, two_hop_call
from .validate import validate
from .validate_micro import validate_micro

CHAIN_SCENARIOS = [
    ("PyTorch chain (measured)", CHAIN_US_PER_ROW),
    ("hypothetical fused target", 0.012),
    ("zero implementation overhead (upper bound)", 0.0),
]
RATIOS = (1.03, 2.0, 3.2, 4.5, 8.0, 15.7)


def comm_speedup(cluster, q: int, tok: int, k_base: int = 6) -> float:
    k = k_base if k_base % q == 0 and k_base >= q else q
    g = MoEGeometry(name="sweep", n_groups=16, R=cluster.R, k=k, M=max(k // q, 1), seq=tok,
                    mbs=1, gbs=16 * cluster.R * tok)
    return one_hop_call(cluster, g) / two_hop_call(cluster, g)


def ratio_table(qs=(2, 3, 6), tok: int = 4096) -> dict:
    """{tier name: {q: [speedup at every ratio of RATIOS]}}"""
    return {name: {q: [comm_speedup(synthetic(r, chain_us_per_row=chain), q, tok)
                       for r in RATIOS] for q in qs}
            for name, chain in CHAIN_SCENARIOS}


def main() -> None:
    cluster = aug_flat()
    t1, _ = validate_micro(cluster, verbose=False)
    print("Tier-1 (communication level): %s" % ("PASS" if t1 else "FAIL"))
    t2, _ = validate(cluster, verbose=False)
    print("Tier-2 (step level): %s" % ("PASS" if t2 else
                                       "FAIL -- step-level extrapolation locked"))
    if not t1:
        raise SystemExit("Tier-1 fails; all extrapolation forbidden.")
    print()
    print("=" * 74)
    print("Communication-level extrapolation (simulation, not measurement)")
    print("x-axis = fast/slow bandwidth ratio; cell = one-hop time / two-hop time "
          "(>1 = two-hop faster)")
    print("Geometry: 16 groups x R=8, k=6, T=4096 tok/rank")
    print("=" * 74)
    table = ratio_table()
    for name, chain in CHAIN_SCENARIOS:
        print("\n-- implementation tier: %s (%.4f us/row) --" % (name, chain))
        print("%-16s" % "q \\ ratio", "".join("%12s" % ("ratio %g" % r) for r in RATIOS))
        for q, cells in table[name].items():
            print("%-16s" % ("q=%d" % q), "".join("%12.2f" % v for v in cells))
    print()
    print("How to read:")
    print("  - The flat column (1.03) stays <=1 at every tier: on a machine without hierarchy")
    print("    the two-hop exchange does not pay for its extra hop.")
    print("  - Columns with ratio >= 3.2 are all >1; the ratios are synthetic scenarios, not")
    print("    target measurements, and the tier changes the magnitude materially.")


if __name__ == "__main__":
    main()
