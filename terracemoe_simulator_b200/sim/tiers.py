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


def measured_cross_supernode_gbps(peers: int) -> float:
    """Marginal bandwidth between the two largest sizes of the peer sweep."""
    t = {(n, b): ms for n, b, ms in PEER_SWEEP}
    lo, hi = 134217728, 268435456
    return (hi - lo) / 2.0 / ((t[(peers, hi)] - t[(peers, lo)]) * 1e-3) / 1e9


def peer_effect_span() -> float:
    vals = [measured_cross_supernode_gbps(n) for n in (1, 2, 4, 8, 16, 32, 64)]
    return max(vals) / min(vals)


@dataclass(frozen=True)
class Topology:
    cards_per_node: int = 8
    nodes_per_supernode: int = 16
    supernodes: int = 2

    @property
    def cards_per_rack(self) -> int:
        return self.cards_per_node * self.nodes_per_supernode


def peer_counts(topo: Topology, world: int, nodes_per_supernode_used: int | None = None) -> dict:
    """How many of a rank's ``world - 1`` peers sit in its node, its supernode, elsewhere."""
    n = topo.cards_per_node
    per_rack = nodes_per_supernode_used if nodes_per_supernode_used is not None else \
        min(topo.nodes_per_supernode, max(1, world // n))
    here = min(world, per_rack * n)
    out = {"intra_node": min(n, world) - 1}
    cross_node = max(0, here - n) if world > n else 0
    if cross_node:
        out["cross_node"] = cross_node
    if world - here > 0:
        out["cross_supernode"] = world - here
    if sum(out.values()) != world - 1:
        raise AssertionError((out, world))
    return out


def compose(peers: dict, tier_gbps: dict) -> float:
    """Harmonic mean of tier bandwidths weighted by peer share (the rejected tier model)."""
    total = sum(peers.values())
    return 1.0 / sum((k / total) / tier_gbps[t] for t, k in peers.items())


def tier_at(tier: str, peers: int) -> float:
    pts = sorted((p, b) for (t, p), b in TIER_BY_PEERS.items() if t == tier)
    if not pts:
        raise ValueError("no measurement for tier %r" % tier)
    if peers < pts[0][0]:
        raise ValueError("%s is measured down to %d peers; %d is the regime Hop A runs in and "
                         "there is no evidence there" % (tier, pts[0][0], peers))
    if peers >= pts[-1][0]:
        return pts[-1][1]
    for (p0, b0), (p1, b1) in zip(pts, pts[1:]):
        if p0 <= peers <= p1:
            w = (math.log(peers) - math.log(p0)) / (math.log(p1) - math.log(p0))
            return b0 + w * (b1 - b0)
    return pts[-1][1]


def hop_a_peer_count(n_groups: int) -> int:
    return max(n_groups - 1, 1)


def main() -> None:
    topo = Topology()
    print("peer counts by tier:")
    for label, world, used in (("world 8, one node", 8, 1),
                               ("world 16, two nodes one supernode", 16, 2),
                               ("world 16, one node per supernode", 16, 1),
                               ("world 128, 8 nodes per supernode", 128, 8),
                               ("world 128, one full supernode", 128, 16)):
        print("  %-36s %s" % (label, peer_counts(topo, world, used)))
    miss = OUT_OF_SAMPLE["predicted_gbps"] / OUT_OF_SAMPLE["measured_gbps"] - 1
    print("tier composition out of sample: predicted %.1f GB/s, measured %.1f (%+.0f%%): rejected"
          % (OUT_OF_SAMPLE["predicted_gbps"], OUT_OF_SAMPLE["measured_gbps"], 100 * miss))
    print("cross-supernode bandwidth by peer count:")
    for n in (1, 2, 4, 8, 16, 32, 64):
        print("  %2d peers  %.1f GB/s" % (n, measured_cross_supernode_gbps(n)))
    print("span %.2fx; uncontended 8 peers %.1f GB/s against %.1f under load"
          % (peer_effect_span(), CROSS_SUPERNODE_8_PEERS_UNCONTENDED,
             TIER_BY_PEERS[("cross_supernode", 8)]))
    for ng in (2, 4, 16):
        note = "   below anything measured" if hop_a_peer_count(ng) < 8 else ""
        print("  Hop A with %2d groups talks to %2d peers%s" % (ng, hop_a_peer_count(ng), note))


if __name__ == "__main__":
    main()
