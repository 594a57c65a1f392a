"""B200 gate: the calibrated cost model against the measured two-hop / one-hop time ratios.

The committed sweep (``sim/data/b200_sweep_8gpu.json``: 48 configurations on 8 x B200, fused
transport, R in {1, 2, 4}, q in {1..4}, 256-16384 tokens per GPU) gives a measured ratio for every
configuration; the gate passes when the model's ratio is within 10 % of it in the median and
within 15 % in the worst case.  This is the B200 counterpart of the reference's measured
two-hop check (``sim/twohop_measured.py``), whose model error was 14 % in the median.
"""
from __future__ import annotations

from .calibrate import _sweep_geometry, b200_nvswitch, load_b200_sweep
from .core import one_hop_call, two_hop_call

GATE_MEDIAN = 0.10
GATE_WORST = 0.15


def validate_b200(cluster=None, rows=None, verbose: bool = True):
    cluster = cluster or b200_nvswitch()
    rows = rows if rows is not None else load_b200_sweep()
    out, errs = [], []
    for r in rows:
        g = _sweep_geometry(r)
        one, two = one_hop_call(cluster, g), two_hop_call(cluster, g)
        measured = r["two_hop_ms"] / r["one_hop_ms"]
        err = (two / one - measured) / measured
        errs.append(abs(err))
        out.append((r["R"], r["q"], r["tokens"], r["one_hop_ms"], 2 * one, r["two_hop_ms"],
                    2 * two, measured, two / one, err))
    ordered = sorted(errs)
    median, worst = ordered[len(ordered) // 2], ordered[-1]
    ok = median <= GATE_MEDIAN and worst <= GATE_WORST
    if verbose:
        print("B200 gate: model two-hop/one-hop ratio vs measured, %d configurations" % len(rows))
        print("%2s %2s %6s  %9s %9s  %9s %9s  %7s %7s %7s" % ("R", "q", "tok", "1hop ms", "model",
                                                              "2hop ms", "model", "ratio", "model",
                                                              "err"))
        for R, q, tok, m1, p1, m2, p2, rm, rp, e in out:
            print("%2d %2d %6d  %9.3f %9.3f  %9.3f %9.3f  %7.3f %7.3f %+6.1f%%"
                  % (R, q, tok, m1, p1, m2, p2, rm, rp, e * 100))
        print("ratio error: median %.1f%% (gate %.0f), worst %.1f%% (gate %.0f)"
              % (median * 100, GATE_MEDIAN * 100, worst * 100, GATE_WORST * 100))
        print("**B200 gate %s**" % ("PASS" if ok else "FAIL"))
    return ok, {"median": median, "worst": worst, "rows": out}


def main() -> None:
    validate_b200()


if __name__ == "__main__":
    main()
