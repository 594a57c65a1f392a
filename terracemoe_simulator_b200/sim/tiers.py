"""Topology tiers of platform A: exact peer counting per tier, a harmonic composition of tier
bandwidths (tried and REJECTED: it misses the world-128 cross-supernode measurement by 31 %), and
the direct cross-supernode peer sweep (peer count barely matters: under 10 % from 1 to 64 peers).

Parity with the reference ``sim/tiers.py`` (:105-233).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

from .records import PEER_SWEEP

TIER_BY_PEERS = {("intra_node", 7): 101.1, ("cross_node", 8): 103.0, ("cross_node", 120): 118.9,
                 ("cross_supernode", 8): 13.3, ("cross_supernode", 64): 20.0}
CROSS_SUPERNODE_8_PEERS_UNCONTENDED = 25.9
OUT_OF_SAMPLE = {"config": "world 128 across both supernodes", "predicted_gbps": 23.4,
                 "measured_gbps": 33.9}


SWEEP_PEERS = (1, 2, 4, 8, 16, 32, 64)
_TOP_TWO_SIZES = (128 << 20, 256 << 20)


def measured_cross_supernode_gbps(peers: int) -> float:
    """Marginal bandwidth between the two largest sizes of the peer sweep (each rank sends and
    receives half of the added bytes across the boundary)."""
    ms_at = {size: ms for n, size, ms in PEER_SWEEP if n == peers}
    small, large = _TOP_TWO_SIZES
    added_bytes = 0.5 * (large - small)
    added_seconds = 1e-3 * (ms_at[large] - ms_at[small])
    return 1e-9 * added_bytes / added_seconds


def peer_effect_span() -> float:
    rates = list(map(measured_cross_supernode_gbps, SWEEP_PEERS))
    return max(rates) / min(rates)


@dataclass(frozen=True)
class Topology:
    cards_per_node: int = 8
    nodes_per_supernode: int = 16
    supernodes: int = 2

    @property
    def cards_per_rack(self) -> int:
        return self.nodes_per_supernode * self.cards_per_node


def peer_counts(topo: Topology, world: int, nodes_per_supernode_used: int | None = None) -> dict:
    """How many of a rank's ``world - 1`` peers sit in its node, its supernode, elsewhere.
    Tiers without peers are left out."""
    node = topo.cards_per_node
    if nodes_per_supernode_used is None:
        nodes_per_supernode_used = min(max(world // node, 1), topo.nodes_per_supernode)
    in_supernode = min(nodes_per_supernode_used * node, world)
    in_node = min(node, world)
    counts = {"intra_node": in_node - 1, "cross_node": in_supernode - in_node,
              "cross_supernode": world - in_supernode}
    assert sum(counts.values()) == world - 1, (counts, world)
    return {tier: n for tier, n in counts.items() if n > 0 or tier == "intra_node"}


def compose(peers: dict, tier_gbps: dict) -> float:
    """Harmonic mean of tier bandwidths weighted by peer share (the rejected tier model)."""
    everyone = float(sum(peers.values()))
    seconds_per_gb = sum(n / everyone / tier_gbps[tier] for tier, n in peers.items())
    return 1.0 / seconds_per_gb


def tier_at(tier: str, peers: int) -> float:
    """Measured bandwidth of ``tier`` at ``peers`` peers: log-linear between measured counts,
    constant above the largest, refused below the smallest."""
    known = sorted((n, gbps) for (name, n), gbps in TIER_BY_PEERS.items() if name == tier)
    if not known:
        raise ValueError("no measurement for tier %r" % tier)
    fewest, most = known[0], known[-1]
    if peers < fewest[0]:
        raise ValueError("%s is measured down to %d peers; %d is the regime Hop A runs in and "
                         "there is no evidence there" % (tier, fewest[0], peers))
    if peers >= most[0]:
        return most[1]
    for (n0, g0), (n1, g1) in zip(known, known[1:]):
        if n0 <= peers <= n1:
            frac = math.log(peers / n0) / math.log(n1 / n0)
            return g0 + (g1 - g0) * frac
    return most[1]


def hop_a_peer_count(n_groups: int) -> int:
    return max(1, n_groups - 1)


LAYOUTS = (("world 8, one node", 8, 1), ("world 16, two nodes one supernode", 16, 2),
           ("world 16, one node per supernode", 16, 1),
           ("world 128, 8 nodes per supernode", 128, 8), ("world 128, one full supernode", 128, 16))


def main() -> None:
    rack = Topology()
    print("peer counts by tier:")
    for label, world, nodes_used in LAYOUTS:
        print("  %-36s %s" % (label, peer_counts(rack, world, nodes_used)))
    predicted, measured = OUT_OF_SAMPLE["predicted_gbps"], OUT_OF_SAMPLE["measured_gbps"]
    print("tier composition out of sample: predicted %.1f GB/s, measured %.1f (%+.0f%%): rejected"
          % (predicted, measured, 100.0 * (predicted / measured - 1.0)))
    print("cross-supernode bandwidth by peer count:")
    print("\n".join("  %2d peers  %.1f GB/s" % (n, measured_cross_supernode_gbps(n))
                    for n in SWEEP_PEERS))
    print("span %.2fx; uncontended 8 peers %.1f GB/s against %.1f under load"
          % (peer_effect_span(), CROSS_SUPERNODE_8_PEERS_UNCONTENDED,
             TIER_BY_PEERS["cross_supernode", 8]))
    for groups in (2, 4, 16):
        talks_to = hop_a_peer_count(groups)
        print("  Hop A with %2d groups talks to %2d peers%s"
              % (groups, talks_to, "   below anything measured" if talks_to < 8 else ""))


if __name__ == "__main__":
    main()
