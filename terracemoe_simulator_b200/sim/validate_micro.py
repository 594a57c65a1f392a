"""Tier-1 gate: the communication-level model against pooled micro measurements.

Targets are pure-communication medians (no splits read-back, no arrival chain) of the one-hop
and the two-hop exchange on 16 groups x 8 ranks, k = 6, M = 2, H = 2048.  The gate passes when
the median relative error is at most 20 %, the worst at most 35 %, and the predicted
one-hop/two-hop crossover falls inside [2048, 16384] tokens per rank.

Parity with the reference ``sim/validate_micro.py`` (targets :36-42, gate :45-83).
"""
from __future__ import annotations

import dataclasses

from .core import MoEGeometry, one_hop_call, two_hop_call

# (tokens per rank, one-hop ms, two-hop ms, number of pooled runs)
MICRO_TARGETS = [(256, 0.394, 0.340, 4), (1024, 0.639, 0.510, 2), (2048, 0.856, 0.670, 4),
                 (4096, 1.366, 1.217, 4), (8192, 2.119, 2.360, 2)]
GATE_MEDIAN, GATE_WORST, GATE_CROSS = 0.20, 0.35, (2048, 16384)


def _geometry(tokens: int) -> MoEGeometry:
    return MoEGeometry(name="micro", n_groups=16, R=8, k=6, M=2, seq=tokens, mbs=1,
                       gbs=16 * 8 * tokens)


def validate_micro(cluster, verbose: bool = True):
    comm_only = dataclasses.replace(cluster, splits_sync_ms=0.0, chain_us_per_row=0.0)
    rows, errors = [], []
    for tokens, one_ms, two_ms, runs in MICRO_TARGETS:
        g = _geometry(tokens)
        p1, p2 = one_hop_call(comm_only, g), two_hop_call(comm_only, g)
        e1, e2 = (p1 - one_ms) / one_ms, (p2 - two_ms) / two_ms
        errors += [abs(e1), abs(e2)]
        rows.append((tokens, one_ms, p1, e1, two_ms, p2, e2, runs))
    ordered = sorted(errors)
    median, worst = ordered[len(ordered) // 2], ordered[-1]
    cross = (None, None)
    last = None
    for tokens in (1024, 2048, 4096, 8192, 16384):
        g = _geometry(tokens)
        ratio = one_hop_call(comm_only, g) / two_hop_call(comm_only, g)
        if last is not None and (last[1] - 1.0) * (ratio - 1.0) < 0:
            cross = (last[0], tokens)
        last = (tokens, ratio)
    cross_ok = cross[0] is not None and cross[0] >= GATE_CROSS[0] and cross[1] <= GATE_CROSS[1]
    ok = median <= GATE_MEDIAN and worst <= GATE_WORST and cross_ok
    if verbose:
        print("Tier-1 (communication micro level) vs pooled multi-run medians")
        print("%6s %4s  %8s %8s %7s   %8s %8s %7s" % ("tok", "runs", "1hop ms", "pred", "err",
                                                      "2hop ms", "pred", "err"))
        for tokens, m1, p1, e1, m2, p2, e2, runs in rows:
            print("%6d %4d  %8.3f %8.3f %+6.1f%%   %8.3f %8.3f %+6.1f%%"
                  % (tokens, runs, m1, p1, e1 * 100, m2, p2, e2 * 100))
        where = "%s-%s" % cross if cross[0] else "no crossing"
        print("relative error: median %.1f%% (gate 20), worst %.1f%% (gate 35); crossover %s "
              "(gate [2048,16384])" % (median * 100, worst * 100, where))
        print("**Tier-1 %s**" % ("PASS -- communication-level extrapolation allowed" if ok
                                 else "FAIL"))
    return ok, {"median": median, "worst": worst, "cross": cross, "rows": rows}


if __name__ == "__main__":
    from .calibrate import flat_supernode
    validate_micro(flat_supernode())
