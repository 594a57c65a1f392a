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
REMOTE_PEERS, LOCAL_PEERS = 8, 7          # of the 15 peers of a rank at world 16


def _seconds_per_byte(points) -> float:
    """Least-squares slope of seconds against bytes over ``points`` = [(bytes, seconds)]."""
    n = float(len(points))
    sx = sum(b for b, _ in points)
    sy = sum(t for _, t in points)
    sxx = sum(b * b for b, _ in points)
    sxy = sum(b * t for b, t in points)
    return (n * sxy - sx * sy) / (n * sxx - sx * sx)


def marginal_gbps(config: str, style: str, n_top: int = 4) -> float:
    """Bandwidth read off the slope of time against wire bytes over the ``n_top`` largest sizes
    (the intercept absorbs the fixed cost, so this is the marginal rate)."""
    column = _COLUMN[config, style]
    wire_share = (WORLD - 1) / WORLD
    largest = sorted(MEASURED)[-n_top:]
    return 1e-9 / _seconds_per_byte([(wire_share * row[0], 1e-3 * row[column]) for row in largest])


def hierarchy_ratio(style: str = "percall", n_top: int = 4) -> float:
    within, across = (marginal_gbps(side, style, n_top) for side in ("within", "across"))
    return within / across


def remote_tier_gbps(config: str, style: str = "percall") -> float:
    """Bandwidth of the eight remote peers alone: the time per byte of the mixed exchange minus
    the share the seven intra-node peers account for at their own rate."""
    peers = WORLD - 1
    mixed_s_per_gb = 1.0 / marginal_gbps(config, style)
    local_s_per_gb = (LOCAL_PEERS / peers) / INTRA_NODE_GBPS
    return (REMOTE_PEERS / peers) / (mixed_s_per_gb - local_s_per_gb)


def contention_penalty() -> float:
    per_card = dict(CONTENTION)
    return per_card[min(per_card)] / per_card[max(per_card)]


def loaded_ratio(pair: str = "pool110/pool111") -> float:
    from .calibrate import BETA_FLAT
    return BETA_FLAT / CROSS_SUPERNODE_WORLD128_GBPS[pair]


def shallowest_boundary() -> float:
    return min(map(loaded_ratio, CROSS_SUPERNODE_WORLD128_GBPS))


def clears_at_hidden_width() -> list:
    from .uncertainty import breakeven_vs_hidden_width
    boundary = shallowest_boundary()
    return [(H, needed, needed <= boundary) for H, needed in breakeven_vs_hidden_width()]


def byte_breakeven_at_supernode(q: int) -> float:
    from .profile import byte_breakeven
    return byte_breakeven(CARDS_PER_SUPERNODE, q)


def placement() -> dict:
    """Where the measured world-16 ratio sits among the break-even ratios of the three chain
    tiers; ``decided_by_the_chain`` is true when it clears the fused tier but not the measured
    PyTorch chain."""
    from .sweep import CHAIN_SCENARIOS
    from .uncertainty import breakeven_ratio
    measured = hierarchy_ratio()
    needed = {tier: breakeven_ratio(chain) for tier, chain in CHAIN_SCENARIOS}
    clears = {tier: value <= measured for tier, value in needed.items()}
    between = clears["hypothetical fused target"] and not clears["PyTorch chain (measured)"]
    return {"ratio": measured, "thresholds": needed, "clears": clears,
            "decided_by_the_chain": between}


def main() -> None:
    from .calibrate import BETA_FLAT
    say = print
    say("CONTENTION: identical work per pair, only the number of crossing pairs moves")
    for pairs, gbps in CONTENTION:
        say("   %d pair(s) crossing   %5.1f GB/s per card" % (pairs, gbps))
    say("   penalty once you are not alone: %.2fx\n" % contention_penalty())
    say("LOADED HIERARCHY RATIO, like-for-like at world 128:")
    say("   within one supernode   %5.1f GB/s" % BETA_FLAT)
    for pair in sorted(CROSS_SUPERNODE_WORLD128_GBPS):
        say("   across %-18s %5.1f GB/s   ratio %5.2f"
            % (pair, CROSS_SUPERNODE_WORLD128_GBPS[pair], loaded_ratio(pair)))
    say("   against the measured-chain threshold, by hidden width:")
    for H, needed, cleared in clears_at_hidden_width():
        say("      H=%5d  threshold %.2f   %s" % (H, needed, "CLEARED" if cleared else "not cleared"))
    say("\n%-18s %14s %14s" % ("world 16", "burst", "percall"))
    for side, label in (("within", "within supernode"), ("across", "across supernodes")):
        say("%-18s %9.1f GB/s %9.1f GB/s" % ((label,) + tuple(marginal_gbps(side, style)
                                                              for style in ("burst", "percall"))))
    say("%-18s %14.2f %14.2f" % ("ratio", hierarchy_ratio("burst"), hierarchy_ratio("percall")))
    tier_in, tier_out = remote_tier_gbps("within"), remote_tier_gbps("across")
    say("pure remote tiers: %.1f GB/s within, %.1f across, ratio %.2f"
        % (tier_in, tier_out, tier_in / tier_out))
    where = placement()
    say("\nbyte-only criterion with a supernode as the fast domain (R = %d): q=2 needs %.2f, q=3 "
        "needs %.2f" % ((CARDS_PER_SUPERNODE,) + tuple(map(byte_breakeven_at_supernode, (2, 3)))))
    for tier, needed in where["thresholds"].items():
        say("   %-44s %.2f   %s" % (tier, needed, "cleared" if where["clears"][tier] else "not cleared"))
    say("   measured supernode boundary                       %.2f" % where["ratio"])
    say("Not an end-to-end verdict: alpha above world 128 is unsupported.")


if __name__ == "__main__":
    main()
