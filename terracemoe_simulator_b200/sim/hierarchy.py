"""The measured hierarchy of platform A: supernode boundary tables and the ratios they give.

World 16 both ways (eight ranks on each of two nodes); the only difference between the two
configurations is whether the eight remote peers sit in the same supernode.  Marginal bandwidth
(slope over the largest sizes) gives a hierarchy ratio of 2.55-2.58; the like-for-like loaded
ratios at world 128 are 5.10 and 7.51 (23.1 / 15.7 GB/s against 117.8).

Parity with the reference ``sim/hierarchy.py`` (:155-317).
"""
from __future__ import annotations

from .records import ACROSS_SUPERNODE, HOST_REGIME, SIZES_23

# (bytes, within burst, within per-call, across burst, across per-call) in ms
MEASURED = [(b, HOST_REGIME[16]["burst"][i], HOST_REGIME[16]["percall"][i],
             ACROSS_SUPERNODE["burst"][i], ACROSS_SUPERNODE["percall"][i])
            for i, b in enumerate(SIZES_23)]
WORLD = 16
CARDS_PER_SUPERNODE = 128
INTRA_NODE_GBPS = 122.4
INTRA_NODE_MEASURED_GBPS = 101.1
CONTENTION = [(1, 39.7), (2, 22.2), (4, 22.1), (8, 22.4)]     # (crossing pairs, GB/s per card)
CROSS_SUPERNODE_WORLD128_GBPS_THREE_POINT_FIT = 33.9
CROSS_SUPERNODE_WORLD128_GBPS = {"pool110/pool111": 23.1, "pool110/pool12": 15.7}
LOADED_RATIO = {"pool110/pool111": 5.10, "pool110/pool12": 7.51}
BOUNDARIES_DIFFER_BY = 1.48
RATIO_BURST, RATIO_PERCALL = 2.58, 2.55
TIER_WITHIN_RACK_GBPS, TIER_ACROSS_SUPERNODE_GBPS, TIER_RATIO = 89.2, 25.2, 3.54
_COLUMN = {("within", "burst"): 1, ("within", "percall"): 2, ("across", "burst"): 3,
           ("across", "percall"): 4}


def marginal_gbps(config: str, style: str, n_top: int = 4) -> float:
    col = _COLUMN[(config, style)]
    pts = sorted(MEASURED)[-n_top:]
    xs = [r[0] * (WORLD - 1) / WORLD for r in pts]
    ys = [r[col] * 1e-3 for r in pts]
    mx, my = sum(xs) / len(xs), sum(ys) / len(ys)
    slope = sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / sum((x - mx) ** 2 for x in xs)
    return 1.0 / slope / 1e9


def hierarchy_ratio(style: str = "percall", n_top: int = 4) -> float:
    return marginal_gbps("within", style, n_top) / marginal_gbps("across", style, n_top)


def remote_tier_gbps(config: str, style: str = "percall") -> float:
    """Bandwidth of the eight remote peers alone, the seven intra-node peers deconvolved."""
    eff = marginal_gbps(config, style)
    intra_share = (7.0 / (WORLD - 1)) / INTRA_NODE_GBPS
    return (8.0 / (WORLD - 1)) / (1.0 / eff - intra_share)


def contention_penalty() -> float:
    d = dict(CONTENTION)
    return d[1] / d[8]


def loaded_ratio(pair: str = "pool110/pool111") -> float:
    from .calibrate import BETA_FLAT
    return BETA_FLAT / CROSS_SUPERNODE_WORLD128_GBPS[pair]


def shallowest_boundary() -> float:
    return min(loaded_ratio(p) for p in CROSS_SUPERNODE_WORLD128_GBPS)


def clears_at_hidden_width() -> list:
    from .uncertainty import breakeven_vs_hidden_width
    r = shallowest_boundary()
    return [(H, be, r >= be) for H, be in breakeven_vs_hidden_width()]


def byte_breakeven_at_supernode(q: int) -> float:
    from .profile import byte_breakeven
    return byte_breakeven(CARDS_PER_SUPERNODE, q)


def placement() -> dict:
    from .sweep import CHAIN_SCENARIOS
    from .uncertainty import breakeven_ratio
    th = {name: breakeven_ratio(chain) for name, chain in CHAIN_SCENARIOS}
    r = hierarchy_ratio()
    return {"ratio": r, "thresholds": th, "clears": {n: r >= v for n, v in th.items()},
            "decided_by_the_chain": (r < th["PyTorch chain (measured)"]
                                     and r >= th["hypothetical fused target"])}


def main() -> None:
    from .calibrate import BETA_FLAT
    print("CONTENTION: identical work per pair, only the number of crossing pairs moves")
    for n, bw in CONTENTION:
        print("   %d pair(s) crossing   %5.1f GB/s per card" % (n, bw))
    print("   penalty once you are not alone: %.2fx" % contention_penalty())
    print()
    print("LOADED HIERARCHY RATIO, like-for-like at world 128:")
    print("   within one supernode   %5.1f GB/s" % BETA_FLAT)
    for pair, bw in sorted(CROSS_SUPERNODE_WORLD128_GBPS.items()):
        print("   across %-18s %5.1f GB/s   ratio %5.2f" % (pair, bw, loaded_ratio(pair)))
    print("   against the measured-chain threshold, by hidden width:")
    for H, be, ok in clears_at_hidden_width():
        print("      H=%5d  threshold %.2f   %s" % (H, be, "CLEARED" if ok else "not cleared"))
    print()
    print("%-18s %14s %14s" % ("world 16", "burst", "percall"))
    for cfg, label in (("within", "within supernode"), ("across", "across supernodes")):
        print("%-18s %9.1f GB/s %9.1f GB/s" % (label, marginal_gbps(cfg, "burst"),
                                               marginal_gbps(cfg, "percall")))
    print("%-18s %14.2f %14.2f" % ("ratio", hierarchy_ratio("burst"), hierarchy_ratio("percall")))
    print("pure remote tiers: %.1f GB/s within, %.1f across, ratio %.2f"
          % (remote_tier_gbps("within"), remote_tier_gbps("across"),
             remote_tier_gbps("within") / remote_tier_gbps("across")))
    p = placement()
    print()
    print("byte-only criterion with a supernode as the fast domain (R = %d): q=2 needs %.2f, q=3 "
          "needs %.2f" % (CARDS_PER_SUPERNODE, byte_breakeven_at_supernode(2),
                          byte_breakeven_at_supernode(3)))
    for name, v in p["thresholds"].items():
        print("   %-44s %.2f   %s" % (name, v, "cleared" if p["clears"][name] else "not cleared"))
    print("   measured supernode boundary                       %.2f" % p["ratio"])
    print("Not an end-to-end verdict: alpha above world 128 is unsupported.")


if __name__ == "__main__":
    main()
