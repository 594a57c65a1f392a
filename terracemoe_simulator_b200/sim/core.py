"""Cost-model core: communication levels, cluster and MoE geometry, per-call cost of the one-hop
and the two-hop dispatch, per-step composition.

    t_a2a [ms] = alpha(world) + wire_bytes / beta(per_peer_bytes)

``alpha`` is piecewise linear in the world size, ``beta`` piecewise linear in log(bytes), both
clamped outside their tables.  Of the rows of an exchange a ``self_fraction`` never crosses the
link.  One-hop: level ``flat``, world EP, T*k rows, self 1/EP.  Two-hop: Hop A on ``slow`` with
world N_g, T*M rows, self 1/N_g; Hop B on ``fast`` with world R, T*k rows, self 1/R; plus one
splits read-back and the arrival chain per (row, pick) pair.  ``hop_overlap`` (new, 0 by default)
prices the two hops as partly concurrent, for transports that pipeline them.

Parity with the reference ``sim/core.py``: ``Level`` :21-60, ``ClusterSpec`` :63-115,
``MoEGeometry`` :122-178, ``_a2a_ms`` :185-217, ``one_hop_call`` :220-224,
``hop_a_self_fraction`` :227-237, ``two_hop_call`` :240-258, ``step_delta`` :261-277.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

OPERATING_POINT_BYTES = 8 * 2 ** 20     # where ClusterSpec.ratio() compares the levels


def _interp(points, x: float, logx: bool = False) -> float:
    """Piecewise-linear lookup in ``[(x, y), ...]`` (ascending x), clamped at both ends;
    ``logx`` interpolates along log(x)."""
    if not points:
        raise ValueError("empty interpolation table: the level was never calibrated")
    first, last = points[0], points[-1]
    if not x > first[0]:
        return first[1]
    if not x < last[0]:
        return last[1]
    axis = math.log if logx else float
    for (xa, ya), (xb, yb) in zip(points, points[1:]):
        if xa <= x <= xb:
            t = (axis(x) - axis(xa)) / (axis(xb) - axis(xa))
            return ya + t * (yb - ya)
    return last[1]


@dataclass
class Level:
    """One communication domain: fixed cost per exchange and bandwidth per message size."""
    name: str
    alpha_pts: list = field(default_factory=list)    # [(world, ms)]
    beta_pts: list = field(default_factory=list)     # [(per-peer bytes, GB/s)]

    def alpha_ms(self, world: int) -> float:
        return _interp(self.alpha_pts, float(world))

    def beta_gbps(self, per_peer_bytes: float) -> float:
        return _interp(self.beta_pts, per_peer_bytes, logx=True)

    def peak_gbps(self) -> float:
        """Bandwidth of the largest tabulated message."""
        return self.beta_gbps(math.inf)


@dataclass
class ClusterSpec:
    """A machine: ``fast`` inside a group of R ranks, ``slow`` between groups, ``flat`` what a
    one-hop exchange over all ranks effectively sees."""
    name: str
    R: int
    fast: Level
    slow: Level
    flat: Level
    splits_sync_ms: float = 0.044
    chain_us_per_row: float = 1.042 * 1000.0 / 24576.0
    combine_exponent: float = 1.0       # p of (alpha^p + T^p)^(1/p); 1 = additive
    per_peer_us: float = 0.0            # explicit cost per peer message (replaces the beta curve)
    hop_overlap: float = 0.0            # 0 = hops strictly serial, 1 = fully overlapped
    self_copy_gbps: float = 0.0         # > 0: rows that stay on the rank cost a local copy
    self_overlap_p: float = 1.0         # wire and local copy combine as (w^p + l^p)^(1/p)

    def ratio(self) -> float:
        at = OPERATING_POINT_BYTES
        return self.fast.beta_gbps(at) / self.slow.beta_gbps(at)

    def price(self, level: Level, world: int, rows: float, row_bytes: int, stays: float) -> float:
        """One exchange on ``level`` with this machine's combination rules."""
        return _a2a_ms(level, world, rows, row_bytes, stays, self.combine_exponent,
                       self.per_peer_us, self.self_copy_gbps, self.self_overlap_p)


@dataclass
class MoEGeometry:
    name: str
    n_groups: int
    R: int
    k: int
    M: int
    H: int = 2048
    seq: int = 4096
    mbs: int = 1
    gbs: int = 512
    moe_layers: int = 19
    bytes_per_elem: int = 2

    @property
    def q(self) -> int:
        quota, rest = divmod(self.k, self.M)
        if rest:
            raise ValueError(f"k={self.k} is not a multiple of M={self.M}")
        return quota

    @property
    def ep(self) -> int:
        return self.R * self.n_groups

    @property
    def tokens_per_rank(self) -> int:
        return self.mbs * self.seq

    @property
    def microbatches(self) -> int:
        count, rest = divmod(self.gbs, self.mbs * self.ep)
        if rest:
            raise ValueError(f"gbs={self.gbs} is not divisible by ep*mbs={self.mbs * self.ep}")
        return count

    def calls_per_step_bwd(self) -> int:
        return self.microbatches * self.moe_layers

    def calls_per_step_fwd(self) -> int:                 # dispatch and combine
        return 2 * self.calls_per_step_bwd()

    def row_bytes(self) -> int:
        return self.bytes_per_elem * self.H

    def rows_hop_a(self) -> int:                         # one row per (token, chosen group)
        return self.M * self.tokens_per_rank

    def rows_hop_b(self) -> int:                         # one row per (token, pick)
        return self.k * self.tokens_per_rank

    rows_one_hop = rows_hop_b


def _p_norm(a: float, b: float, p: float) -> float:
    """(a^p + b^p)^(1/p): the plain sum at p = 1, towards max(a, b) as p grows."""
    return a + b if p == 1.0 else (a ** p + b ** p) ** (1.0 / p)


def _a2a_ms(level: Level, world: int, total_rows: float, row_bytes: int, self_fraction: float,
            combine_exponent: float = 1.0, per_peer_us: float = 0.0, self_copy_gbps: float = 0.0,
            self_overlap_p: float = 1.0) -> float:
    """Time of one all-to-all: fixed cost + bytes on the wire over the bandwidth at the per-peer
    message size (or over the peak bandwidth plus an explicit per-message cost), the rows that
    stay on the rank optionally priced as a local copy that partly overlaps the wire."""
    payload = row_bytes * total_rows
    on_wire = payload * (1.0 - self_fraction)
    wire_ms = 0.0
    if on_wire > 0.0:
        if per_peer_us > 0.0:
            wire_ms = on_wire / (1e6 * level.peak_gbps()) + 1e-3 * per_peer_us * (world - 1)
        else:
            per_peer = on_wire / max(1, world - 1)
            wire_ms = on_wire / (1e6 * level.beta_gbps(per_peer))
    if self_copy_gbps > 0.0:
        local_ms = payload * self_fraction / (1e6 * self_copy_gbps)
        wire_ms = _p_norm(wire_ms, local_ms, self_overlap_p)
    return _p_norm(level.alpha_ms(world), wire_ms, combine_exponent)


def one_hop_call(c: ClusterSpec, g: MoEGeometry) -> float:
    return c.price(c.flat, g.ep, g.rows_one_hop(), g.row_bytes(), 1.0 / g.ep)


def hop_a_self_fraction(g: MoEGeometry) -> float:
    """A token emits M Hop A rows of which M/N_g are expected to stay in its own group."""
    return 1.0 / max(g.n_groups, 1)


def two_hop_parts(c: ClusterSpec, g: MoEGeometry) -> dict:
    pairs = g.rows_hop_b()
    return {"hop_a": c.price(c.slow, g.n_groups, g.rows_hop_a(), g.row_bytes(),
                             hop_a_self_fraction(g)),
            "hop_b": c.price(c.fast, g.R, pairs, g.row_bytes(), 1.0 / g.R),
            "splits": c.splits_sync_ms, "chain": 1e-3 * c.chain_us_per_row * pairs}


def two_hop_call(c: ClusterSpec, g: MoEGeometry) -> float:
    part = two_hop_parts(c, g)
    hidden = c.hop_overlap * min(part["hop_a"], part["hop_b"])
    return part["hop_a"] + part["hop_b"] - hidden + part["splits"] + part["chain"]


def step_delta(c: ClusterSpec, g: MoEGeometry) -> dict:
    """Communication time two-hop minus one-hop for a whole training step: dispatch and combine
    mirror each other (x2), backward replays the forward exchanges at half the call count."""
    per_call = {"per_call_on_ms": two_hop_call(c, g), "per_call_off_ms": one_hop_call(c, g)}
    gap = per_call["per_call_on_ms"] - per_call["per_call_off_ms"]
    n_calls = 2 * (g.calls_per_step_bwd() + g.calls_per_step_fwd())
    return {**per_call, "per_call_delta_ms": gap, "calls_per_step": n_calls,
            "step_delta_ms": n_calls * gap}
