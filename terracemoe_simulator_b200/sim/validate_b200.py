"""B200 gate: the calibrated cost model against measured two-hop / one-hop time ratios, scored
on configurations the calibration did not see.

The committed sweeps (``sim/data/b200_sweep_{2,4,8}gpu.json``, written by ``bench/sweep.py``:
fused transport, R in {1, 2, 4}, q in {1..4}, 256-16384 tokens per GPU) give a measured ratio
per configuration.  Three scores are reported:

  in-sample    the shipped constants (fitted on the whole 8-GPU sweep) on that same sweep --
               fit quality, not prediction
  hold-out     constants re-fitted on the 8-GPU rows with groups of 1 or 4 GPUs and at most
               4096 tokens; scored on the rest (groups of 2 GPUs, and every 16384-token row)
  cross-size   the 8-GPU fit applied to the 2- and 4-GPU sweeps, which it never saw

The gate is on the predictions (hold-out and, where the files exist, cross-size): the median
relative error of the ratio within 10 %.  The stricter reading -- every single row within 10 % --
is reported beside it and does not hold: the rows beyond it are 256- and 1024-token calls of
50-200 us, where one slow burst moves the measured ratio by more than that (one such row of the
8-GPU sweep, R = 2, q = 1, 256 tokens, was caught at twice the time of its neighbours and is
kept in the data).  A fourth line per group size scores the other calibration route
(``calibrate.b200_from_records``: one fixed cost and one bandwidth curve per level, fitted with
``fit.fit_beta_pinned`` to the ``flat`` / ``slow`` / ``fast`` frames of the sweep).  It is the
recipe for a machine where only collective-style exchanges can be timed, and on this transport it
is the worse model (median 9-13 %): a frame is a whole one-hop exchange on the level's peer set,
plan and flags included, while Hop A and Hop B share one plan.  It is reported, not gated.  It is the B200 counterpart of the reference's measured two-hop check
(``sim/twohop_measured.py``), whose model error was 14 % in the median.
"""
from __future__ import annotations

import os
import statistics

from . import calibrate as cal
from .core import one_hop_call, two_hop_call

GATE_MEDIAN = 0.10
GATE_WORST = 0.10
HOLDOUT_MAX_TOKENS = 4096
HOLDOUT_TRAIN_GROUP_SIZES = (1, 4)
DATA_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data")


def sweep_path(n_gpus: int) -> str:
    return os.path.join(DATA_DIR, "b200_sweep_%dgpu.json" % n_gpus)


def score(cluster, rows) -> dict:
    """Relative error of the modelled two-hop / one-hop ratio on ``rows``."""
    table, errs = [], []
    for r in rows:
        g = cal._sweep_geometry(r)
        one, two = one_hop_call(cluster, g), two_hop_call(cluster, g)
        measured = r["two_hop_ms"] / r["one_hop_ms"]
        err = (two / one) / measured - 1.0
        errs.append(abs(err))
        table.append((r["R"], r["q"], r["tokens"], r["one_hop_ms"], 2 * one, r["two_hop_ms"],
                      2 * two, measured, two / one, err))
    return {"n": len(rows), "median": statistics.median(errs) if errs else 0.0,
            "worst": max(errs, default=0.0), "rows": table}


def split_holdout(rows):
    train = [r for r in rows if r["R"] in HOLDOUT_TRAIN_GROUP_SIZES
             and r["tokens"] <= HOLDOUT_MAX_TOKENS]
    held = [r for r in rows if r not in train]
    return train, held


def _passes(s: dict) -> bool:
    return s["median"] <= GATE_MEDIAN


def _every_row(s: dict) -> bool:
    return s["worst"] <= GATE_WORST


def beyond(s: dict, limit: float = GATE_WORST) -> list:
    """``(R, q, tokens, err)`` of the rows whose ratio error exceeds ``limit``."""
    return [(r[0], r[1], r[2], r[9]) for r in s["rows"] if abs(r[9]) > limit]


def validate_b200(cluster=None, rows=None, verbose: bool = True):
    """Returns ``(ok, report)``; ``report`` carries the in-sample score under the historical keys
    ``median`` / ``worst`` / ``rows`` and the prediction scores under ``holdout`` and
    ``cross_size``.  ``ok`` is the gate on the predictions."""
    shipped = cluster or cal.b200_nvswitch()
    rows = rows if rows is not None else cal.load_b200_sweep()
    inside = score(shipped, rows)
    report = {"median": inside["median"], "worst": inside["worst"], "rows": inside["rows"],
              "in_sample": inside, "cross_size": {}}
    train, held = split_holdout(rows)
    try:
        refit = cal.b200_from_sweep(train)
    except ImportError:                      # no scipy: the prediction scores cannot be made
        refit = None
    report["holdout"] = score(refit, held) if refit is not None and held else None
    for n in (2, 4):
        if os.path.isfile(sweep_path(n)):
            other = cal.load_b200_sweep(sweep_path(n))
            report["cross_size"][n] = score(shipped, other)
    # the other calibration route: one alpha and one saturating beta per level from the
    # ``flat`` / ``slow`` / ``fast`` frames of the same sweep file (fit.fit_beta_pinned), scored
    # on the rows whose group size the frames were measured with
    report["per_level"] = {}
    try:
        records = cal.load_b200_records()
    except (OSError, KeyError):
        records = []
    for R in sorted({r.get("R") for r in records if r.get("frame") in ("slow", "fast")} - {None}):
        subset = [r for r in rows if r["R"] == R]
        if subset:
            report["per_level"][R] = score(cal.b200_from_records(records, R=R), subset)
    predictions = [s for s in [report["holdout"], *report["cross_size"].values()] if s]
    ok = bool(predictions) and all(_passes(s) for s in predictions)
    report["every_row"] = bool(predictions) and all(_every_row(s) for s in predictions)
    report["beyond"] = [row for s in predictions for row in beyond(s)]
    if verbose:
        print("\n".join(_lines(report, len(train), ok)))
    return ok, report


def _lines(report, n_train, ok) -> list:
    out = ["B200 gate: model two-hop/one-hop ratio vs measured",
           "%2s %2s %6s  %9s %9s  %9s %9s  %7s %7s %7s" % ("R", "q", "tok", "1hop ms", "model",
                                                           "2hop ms", "model", "ratio", "model",
                                                           "err")]
    out += ["%2d %2d %6d  %9.3f %9.3f  %9.3f %9.3f  %7.3f %7.3f %+6.1f%%"
            % (row[:9] + (100 * row[9],)) for row in report["rows"]]

    def line(label, s):
        return "%-34s %3d rows: median %4.1f%%, worst %4.1f%%" % (label, s["n"], 100 * s["median"],
                                                                  100 * s["worst"])
    out.append(line("in-sample (shipped constants)", report["in_sample"]))
    if report["holdout"]:
        out.append(line("hold-out (fit on %d other rows)" % n_train, report["holdout"]))
    for n, s in sorted(report["cross_size"].items()):
        out.append(line("cross-size: %d-GPU sweep" % n, s))
    small = sum(1 for _r, _q, tok, _e in report["beyond"] if tok <= 1024)
    for R, s in sorted(report.get("per_level", {}).items()):
        out.append(line("per-level frames, groups of %d" % R, s))
    out.append("gate on the predictions: median within %.0f %%" % (100 * GATE_MEDIAN))
    out.append("**B200 gate %s**" % ("PASS" if ok else "FAIL"))
    out.append("every predicted row within %.0f %%: %s (%d rows beyond, %d of them at 1024 tokens "
               "or fewer)" % (100 * GATE_WORST, "yes" if report["every_row"] else "no",
                              len(report["beyond"]), small))
    return out


def main() -> None:
    validate_b200()


if __name__ == "__main__":
    main()
