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

import bisect
import math
from dataclasses import dataclass, field

OPERATING_POINT_BYTES = 8 * 2 ** 20     # where ClusterSpec.ratio() compares the levels


def _interp(points, x: float, logx: bool = False) -> float:
    """Piecewise-linear lookup in ``[(x, y), ...]`` (ascending x), clamped at both ends."""
    if not points:
        raise ValueError("empty interpolation table: the level was never calibrated")
    xs = [p[0] for p in points]
    if x <= xs[0]:
        return points[0][1]
    if x >= xs[-1]:
        return points[-1][1]
    hi = bisect.bisect_right(xs, x)
    (x0, y0), (x1, y1) = points[hi - 1], points[hi]
    if logx:
        w = (math.log(x) - math.log(x0)) / (math.log(x1) - math.log(x0))
    else:
        w = (x - x0) / (x1 - x0)
    return y0 + w * (y1 - y0)


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
        p = OPERATING_POINT_BYTES
        return self.fast.beta_gbps(p) / self.slow.beta_gbps(p)


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
        if self.k % self.M:
            raise ValueError(f"k={self.k} is not a multiple of M={self.M}")
        return self.k // self.M

    @property
    def ep(self) -> int:
        return self.n_groups * self.R

    @property
    def tokens_per_rank(self) -> int:
        return self.seq * self.mbs

    @property
    def microbatches(self) -> int:
        per_pass = self.ep * self.mbs
        if self.gbs % per_pass:
            raise ValueError(f"gbs={self.gbs} is not divisible by ep*mbs={per_pass}")
        return self.gbs // per_pass

    def calls_per_step_fwd(self) -> int:
        return self.moe_layers * self.microbatches * 2

    def calls_per_step_bwd(self) -> int:
        return self.moe_layers * self.microbatches

    def row_bytes(self) -> int:
        return self.H * self.bytes_per_elem

    def rows_one_hop(self) -> int:
        return self.tokens_per_rank * self.k

    def rows_hop_a(self) -> int:
        return self.tokens_per_rank * self.M

    def rows_hop_b(self) -> int:
        return self.tokens_per_rank * self.k


def _a2a_ms(level: Level, world: int, total_rows: float, row_bytes: int, self_fraction: float,
            combine_exponent: float = 1.0, per_peer_us: float = 0.0, self_copy_gbps: float = 0.0,
            self_overlap_p: float = 1.0) -> float:
    wire_bytes = total_rows * (1.0 - self_fraction) * row_bytes
    peers = max(world - 1, 1)
    alpha = level.alpha_ms(world)
    if wire_bytes <= 0.0:
        transfer = 0.0
    elif per_peer_us > 0.0:
        transfer = wire_bytes / (level.beta_gbps(1e12) * 1e6) + (world - 1) * per_peer_us / 1000.0
    else:
        transfer = wire_bytes / (level.beta_gbps(wire_bytes / peers) * 1e6)
    if self_copy_gbps > 0.0:
        local = total_rows * self_fraction * row_bytes / (self_copy_gbps * 1e6)
        p = self_overlap_p
        transfer = (transfer ** p + local ** p) ** (1.0 / p)
    if combine_exponent == 1.0:
        return alpha + transfer
    p = combine_exponent
    return (alpha ** p + transfer ** p) ** (1.0 / p)


def one_hop_call(c: ClusterSpec, g: MoEGeometry) -> float:
    return _a2a_ms(c.flat, g.ep, g.rows_one_hop(), g.row_bytes(), 1.0 / g.ep,
                   c.combine_exponent, c.per_peer_us, c.self_copy_gbps, c.self_overlap_p)


def hop_a_self_fraction(g: MoEGeometry) -> float:
    """A token emits M Hop A rows of which M/N_g are expected to stay in its own group."""
    return 1.0 / g.n_groups if g.n_groups > 1 else 1.0


def two_hop_parts(c: ClusterSpec, g: MoEGeometry) -> dict:
    hop_a = _a2a_ms(c.slow, g.n_groups, g.rows_hop_a(), g.row_bytes(), hop_a_self_fraction(g),
                    c.combine_exponent, c.per_peer_us, c.self_copy_gbps, c.self_overlap_p)
    hop_b = _a2a_ms(c.fast, g.R, g.rows_hop_b(), g.row_bytes(), 1.0 / g.R,
                    c.combine_exponent, c.per_peer_us, c.self_copy_gbps, c.self_overlap_p)
    chain = c.chain_us_per_row * g.rows_hop_b() / 1000.0
    return {"hop_a": hop_a, "hop_b": hop_b, "splits": c.splits_sync_ms, "chain": chain}


def two_hop_call(c: ClusterSpec, g: MoEGeometry) -> float:
    p = two_hop_parts(c, g)
    serial = p["hop_a"] + p["hop_b"]
    hops = serial - c.hop_overlap * min(p["hop_a"], p["hop_b"])
    return hops + p["splits"] + p["chain"]


def step_delta(c: ClusterSpec, g: MoEGeometry) -> dict:
    """Communication time two-hop minus one-hop for a whole training step: dispatch and combine
    mirror each other (x2), backward replays the forward exchanges at half the call count."""
    on, off = two_hop_call(c, g), one_hop_call(c, g)
    calls = 2 * (g.calls_per_step_fwd() + g.calls_per_step_bwd())
    return {"per_call_on_ms": on, "per_call_off_ms": off, "per_call_delta_ms": on - off,
            "calls_per_step": calls, "step_delta_ms": (on - off) * calls}
