"""Routing skew: what the busiest peer of an exchange carries beyond the mean.

An exchange finishes when its fullest buffer has drained.  If expert loads vary with coefficient
of variation ``cv``, a buffer that aggregates ``a`` experts varies with ``cv / sqrt(a)``, and the
largest of ``n`` such buffers sits about ``sqrt(2 ln n)`` standard deviations above the mean.
``Exchange`` describes one collective (level, peers, rows, share that stays local, experts
aggregated per buffer) and prices it balanced or skewed; one-hop is one exchange, two-hop is
Hop A plus Hop B plus its fixed and per-row overheads.

Skew favours two-hop: its maxima run over fewer peers and Hop A aggregates q experts per
message.  It is the one modelled effect that points against the arrival chain, and ``sim.core``
does not apply it: the calibration microbenchmarks divide their buffers equally.

Public surface of the reference's ``sim/imbalance.py`` (:54-113).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

CV_EXPERT_MEDIAN = 0.136
CV_EXPERT_RANGE = (0.118, 0.151)


def expected_max_z(n_peers: int) -> float:
    """Leading-order expected maximum of ``n_peers`` standard normals (at least two peers)."""
    return (2.0 * math.log(n_peers if n_peers > 2 else 2)) ** 0.5


def inflation(n_peers: int, cv_expert: float = CV_EXPERT_MEDIAN, aggregate_over: int = 1) -> float:
    spread = cv_expert * (aggregate_over if aggregate_over > 1 else 1) ** -0.5
    return 1.0 + spread * expected_max_z(int(n_peers))


@dataclass(frozen=True)
class Exchange:
    """One all-to-all of a dispatch: who takes part and how much each rank sends."""
    level: object
    peers: int
    rows: float
    local_share: float
    aggregated: int = 1

    def busiest(self, cv: float) -> float:
        return inflation(self.peers, cv, self.aggregated)

    def ms(self, row_bytes: int, cv: float | None = None) -> float:
        from .core import _a2a_ms
        scale = 1.0 if cv is None else self.busiest(cv)
        return _a2a_ms(self.level, self.peers, self.rows * scale, row_bytes, self.local_share)


def exchanges(cluster, geom) -> dict:
    """The three collectives of the two dispatch strategies for one geometry."""
    stay_a = geom.M / geom.n_groups if geom.n_groups > 1 else 1.0
    return {
        "one_hop": Exchange(cluster.flat, geom.ep, geom.rows_one_hop(), 1.0 / geom.ep),
        "hop_a": Exchange(cluster.slow, geom.n_groups, geom.rows_hop_a(), stay_a, geom.q),
        "hop_b": Exchange(cluster.fast, geom.R, geom.rows_hop_b(), 1.0 / geom.R),
    }


def strategy_inflation(ep: int, n_groups: int, R: int, q: int,
                       cv_expert: float = CV_EXPERT_MEDIAN) -> dict:
    shape = {"one_hop": (ep, 1), "hop_a": (n_groups, q), "hop_b": (R, 1)}
    return {name: inflation(n, cv_expert, agg) for name, (n, agg) in shape.items()}


def adjusted_ratio(cluster, geom, cv_expert: float = CV_EXPERT_MEDIAN) -> dict:
    ex, row = exchanges(cluster, geom), geom.row_bytes()
    overhead = cluster.splits_sync_ms + cluster.chain_us_per_row * geom.rows_hop_b() / 1e3

    def ratio(cv):
        two = ex["hop_a"].ms(row, cv) + ex["hop_b"].ms(row, cv) + overhead
        return ex["one_hop"].ms(row, cv) / two

    flat, skew = ratio(None), ratio(cv_expert)
    return {"factors": {name: e.busiest(cv_expert) for name, e in ex.items()},
            "ratio_balanced": flat, "ratio_skewed": skew, "shift": skew - flat}


REPORT_GEOMETRY = dict(name="skew", n_groups=16, R=8, k=6, M=2, seq=4096, mbs=1,
                       gbs=16 * 8 * 4096)
REPORT_HIERARCHIES = (1.03, 2.0, 3.2, 8.0)


def report() -> list:
    """The module's text report as a list of lines."""
    from .calibrate import synthetic
    from .core import MoEGeometry
    from .sweep import CHAIN_SCENARIOS
    geom = MoEGeometry(**REPORT_GEOMETRY)
    factors = strategy_inflation(geom.ep, geom.n_groups, geom.R, geom.q)
    who = {"one_hop": "one-hop  %3d peers           " % geom.ep,
           "hop_a": "Hop A    %3d peers, agg q=%d  " % (geom.n_groups, geom.q),
           "hop_b": "Hop B    %3d peers           " % geom.R}
    out = ["Measured expert load CV %.3f (range %.3f-%.3f, 16 samples)"
           % ((CV_EXPERT_MEDIAN,) + CV_EXPERT_RANGE),
           "Busiest-peer inflation, by collective:"]
    out += ["  %s %.3f" % (who[name], factors[name]) for name in who]
    out += ["", "Effect on the one-hop / two-hop ratio, fused arrival chain:",
            "  %-8s %11s %11s %9s" % ("ratio", "balanced", "with skew", "shift")]
    fused_chain = CHAIN_SCENARIOS[1][1]
    for hierarchy in REPORT_HIERARCHIES:
        r = adjusted_ratio(synthetic(hierarchy, chain_us_per_row=fused_chain), geom)
        out.append("  %-8.2f %11.3f %11.3f %+9.3f"
                   % (hierarchy, r["ratio_balanced"], r["ratio_skewed"], r["shift"]))
    out += ["", "Skew favours two-hop: its maxima run over fewer peers and Hop A aggregates q",
            "experts per message.  core.py does not apply it: the calibration contains no skew."]
    return out


def main() -> None:
    print("\n".join(report()))


if __name__ == "__main__":
    main()
