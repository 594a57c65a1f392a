"""Routing skew: how much the busiest peer inflates an exchange.

With expert-load coefficient of variation ``cv`` the busiest of ``n`` peers carries about
``1 + cv / sqrt(aggregate) * sqrt(2 ln n)`` times the mean.  Skew favours two-hop (its maxima
run over fewer peers and Hop A aggregates q experts per message), the one modelled effect that
points against the arrival chain -- and ``sim.core`` deliberately does not apply it, because the
calibration microbenchmarks divide their buffers equally.

Parity with the reference ``sim/imbalance.py`` (:54-113).
"""
from __future__ import annotations

import math

CV_EXPERT_MEDIAN = 0.136
CV_EXPERT_RANGE = (0.118, 0.151)


def expected_max_z(n_peers: int) -> float:
    return math.sqrt(2.0 * math.log(max(int(n_peers), 2)))


def inflation(n_peers: int, cv_expert: float = CV_EXPERT_MEDIAN, aggregate_over: int = 1) -> float:
    return 1.0 + cv_expert / math.sqrt(max(aggregate_over, 1)) * expected_max_z(n_peers)


def strategy_inflation(ep: int, n_groups: int, R: int, q: int,
                       cv_expert: float = CV_EXPERT_MEDIAN) -> dict:
    return {"one_hop": inflation(ep, cv_expert),
            "hop_a": inflation(n_groups, cv_expert, aggregate_over=q),
            "hop_b": inflation(R, cv_expert)}


def adjusted_ratio(cluster, geom, cv_expert: float = CV_EXPERT_MEDIAN) -> dict:
    from .core import _a2a_ms
    f = strategy_inflation(geom.ep, geom.n_groups, geom.R, geom.q, cv_expert)
    row = geom.row_bytes()

    def one_hop(scale):
        return _a2a_ms(cluster.flat, geom.ep, geom.rows_one_hop() * scale, row, 1.0 / geom.ep)

    def two_hop(sa, sb):
        self_a = geom.M / geom.n_groups if geom.n_groups > 1 else 1.0
        a = _a2a_ms(cluster.slow, geom.n_groups, geom.rows_hop_a() * sa, row, self_a)
        b = _a2a_ms(cluster.fast, geom.R, geom.rows_hop_b() * sb, row, 1.0 / geom.R)
        return a + b + cluster.splits_sync_ms + cluster.chain_us_per_row * geom.rows_hop_b() / 1e3

    balanced = one_hop(1.0) / two_hop(1.0, 1.0)
    skewed = one_hop(f["one_hop"]) / two_hop(f["hop_a"], f["hop_b"])
    return {"factors": f, "ratio_balanced": balanced, "ratio_skewed": skewed,
            "shift": skewed - balanced}


def main() -> None:
    from .calibrate import synthetic
    from .core import MoEGeometry
    from .sweep import CHAIN_SCENARIOS
    g = MoEGeometry(name="skew", n_groups=16, R=8, k=6, M=2, seq=4096, mbs=1, gbs=16 * 8 * 4096)
    f = strategy_inflation(g.ep, g.n_groups, g.R, g.q)
    print("Measured expert load CV %.3f (range %.3f-%.3f, 16 samples)"
          % (CV_EXPERT_MEDIAN, CV_EXPERT_RANGE[0], CV_EXPERT_RANGE[1]))
    print("Busiest-peer inflation, by collective:")
    print("  one-hop  %3d peers            %.3f" % (g.ep, f["one_hop"]))
    print("  Hop A    %3d peers, agg q=%d   %.3f" % (g.n_groups, g.q, f["hop_a"]))
    print("  Hop B    %3d peers            %.3f" % (g.R, f["hop_b"]))
    print("\nEffect on the one-hop / two-hop ratio, fused arrival chain:")
    print("  %-8s %11s %11s %9s" % ("ratio", "balanced", "with skew", "shift"))
    for r in (1.03, 2.0, 3.2, 8.0):
        out = adjusted_ratio(synthetic(r, chain_us_per_row=CHAIN_SCENARIOS[1][1]), g)
        print("  %-8.2f %11.3f %11.3f %+9.3f" % (r, out["ratio_balanced"], out["ratio_skewed"],
                                                 out["shift"]))
    print("\nSkew favours two-hop: its maxima run over fewer peers and Hop A aggregates q")
    print("experts per message.  core.py does not apply it: the calibration contains no skew.")


if __name__ == "__main__":
    main()
