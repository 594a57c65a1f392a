"""Tier-1 gate: the communication-level model against pooled micro measurements.

Targets are pure-communication medians (no splits read-back, no arrival chain) of the one-hop
and the two-hop exchange on 16 groups x 8 ranks, k = 6, M = 2, H = 2048.  The gate passes when
the median relative error is at most 20 %, the worst at most 35 %, and the predicted
one-hop/two-hop crossover falls inside [2048, 16384] tokens per rank.

Parity with the reference ``sim/validate_micro.py`` (targets :36-42, gate :45-83).
"""
from __future__ import annotations

import dataclasses

from ._text import Column, render_table
from .uncertainty import Shape

# (tokens per rank, one-hop ms, two-hop ms, number of pooled runs)
MICRO_TARGETS = [(256, 0.394, 0.340, 4), (1024, 0.639, 0.510, 2), (2048, 0.856, 0.670, 4),
                 (4096, 1.366, 1.217, 4), (8192, 2.119, 2.360, 2)]
GATE_MEDIAN, GATE_WORST, GATE_CROSS = 0.20, 0.35, (2048, 16384)
CROSS_SCAN = (1024, 2048, 4096, 8192, 16384)


def _both_calls(cluster, tokens: int) -> tuple:
    """(one-hop ms, two-hop ms) of the micro geometry: 16 groups x 8, k = 6, M = 2, H = 2048."""
    return Shape(tok=tokens).calls(cluster)


def crossover(cluster) -> tuple:
    """The neighbouring pair of ``CROSS_SCAN`` between which one-hop / two-hop passes 1 (the
    last such pair), or ``(None, None)``."""
    sides = [(t, _both_calls(cluster, t)) for t in CROSS_SCAN]
    found = (None, None)
    for (t0, (a0, b0)), (t1, (a1, b1)) in zip(sides, sides[1:]):
        if (a0 / b0 - 1.0) * (a1 / b1 - 1.0) < 0:
            found = (t0, t1)
    return found


def validate_micro(cluster, verbose: bool = True):
    comm_only = dataclasses.replace(cluster, splits_sync_ms=0.0, chain_us_per_row=0.0)
    rows = []
    for tokens, one_ms, two_ms, runs in MICRO_TARGETS:
        model_one, model_two = _both_calls(comm_only, tokens)
        rows.append((tokens, one_ms, model_one, model_one / one_ms - 1.0,
                     two_ms, model_two, model_two / two_ms - 1.0, runs))
    errors = sorted(abs(e) for row in rows for e in (row[3], row[6]))
    median, worst = errors[len(errors) // 2], errors[-1]
    cross = crossover(comm_only)
    cross_ok = None not in cross and GATE_CROSS[0] <= cross[0] and cross[1] <= GATE_CROSS[1]
    ok = cross_ok and worst <= GATE_WORST and median <= GATE_MEDIAN
    if verbose:
        pct = lambda i: (lambda r: "%+.1f%%" % (100 * r[i]))          # noqa: E731
        cols = [Column("tok", "%6d", lambda r: r[0]), Column("runs", "%4d", lambda r: r[7]),
                Column("1hop ms", "%8.3f", lambda r: r[1]), Column("pred", "%8.3f", lambda r: r[2]),
                Column("err", "%7s", pct(3)), Column("2hop ms", "%8.3f", lambda r: r[4]),
                Column("pred", "%8.3f", lambda r: r[5]), Column("err", "%7s", pct(6))]
        print("Tier-1 (communication micro level) vs pooled multi-run medians")
        print("\n".join(render_table(cols, rows)))
        where = "no crossing" if cross[0] is None else "%s-%s" % cross
        print("relative error: median %.1f%% (gate 20), worst %.1f%% (gate 35); crossover %s "
              "(gate [2048,16384])" % (100 * median, 100 * worst, where))
        print("**Tier-1 %s**" % ("PASS -- communication-level extrapolation allowed" if ok
                                 else "FAIL"))
    return bool(ok), {"median": median, "worst": worst, "cross": cross, "rows": rows}


if __name__ == "__main__":
    from .calibrate import flat_supernode
    validate_micro(flat_supernode())
