"""Tier-2 gate: predicted end-to-end ``G = t(one-hop step) / t(two-hop step)`` against seven
measured geometries.  One geometry (``flag``) calibrates a per-call combine-side constant, the
other six are held out.  The gate wants MAE <= 0.025, at least four holdouts within +-0.035 and
the sign of all four known-negative geometries right.  With the shipped calibration this gate
FAILS, and that negative result is itself pinned by the tests: step-level extrapolation stays
locked until an overlap model explains the step ledger.

Parity with the reference ``sim/validate.py`` (``HOLDOUTS`` :47-57, ``predict_g`` :60-77,
``calibrate_combine`` :80-92, ``validate`` :95-123).
"""
from __future__ import annotations

from dataclasses import dataclass

from .core import MoEGeometry, step_delta

GATE_MAE, GATE_TOL, GATE_IN_TOL = 0.025, 0.035, 4
NEGATIVE = ("tok2x", "tok4x", "k8m4", "n8")
PAIRS_AT_CALIBRATION = 24576.0


@dataclass
class Holdout:
    geom: MoEGeometry
    t_off_ms: float       # measured step time of the one-hop arm
    g_measured: float
    role: str             # "calibration" | "holdout"


def _geom(name, n_groups, R, k, M, mbs, layers=19) -> MoEGeometry:
    return MoEGeometry(name=name, n_groups=n_groups, R=R, k=k, M=M, mbs=mbs, moe_layers=layers)


HOLDOUTS = [
    Holdout(_geom("flag", 16, 8, 6, 2, 1), 4420.4, 1.0355, "calibration"),
    Holdout(_geom("tok2x", 16, 8, 6, 2, 2), 3343.6, 0.8845, "holdout"),
    Holdout(_geom("tok4x", 16, 8, 6, 2, 4), 2992.7, 0.8234, "holdout"),
    Holdout(_geom("k8m2", 16, 8, 8, 2, 1), 4791.7, 0.9935, "holdout"),
    Holdout(_geom("k8m4", 16, 8, 8, 4, 1), 4664.9, 0.9335, "holdout"),
    Holdout(_geom("n8", 8, 8, 6, 2, 1), 6657.5, 0.9027, "holdout"),
    Holdout(_geom("n4", 4, 8, 6, 2, 1), 11712.0, 0.8647, "holdout"),
]


def _deltas(cluster, h: Holdout):
    d = step_delta(cluster, h.geom)
    calls = h.geom.calls_per_step_fwd() + h.geom.calls_per_step_bwd()
    chain_ms = cluster.chain_us_per_row * h.geom.rows_hop_b() / 1000.0
    dispatch = d["per_call_on_ms"] - d["per_call_off_ms"]          # with the arrival chain
    combine = d["per_call_on_ms"] - chain_ms - d["per_call_off_ms"]  # the return leg has none
    return calls, dispatch, combine


def predict_g(cluster, h: Holdout, combine_extra_ms: float) -> float:
    calls, dispatch, combine = _deltas(cluster, h)
    scale = h.geom.rows_hop_b() / PAIRS_AT_CALIBRATION
    t_on = h.t_off_ms + dispatch * calls + (combine + combine_extra_ms * scale) * calls
    return h.t_off_ms / t_on


def calibrate_combine(cluster) -> float:
    """Per-call combine-side constant that makes the calibration geometry exact."""
    h = next(x for x in HOLDOUTS if x.role == "calibration")
    calls, dispatch, combine = _deltas(cluster, h)
    target_on = h.t_off_ms / h.g_measured
    return (target_on - h.t_off_ms - dispatch * calls) / calls - combine


def validate(cluster, verbose: bool = True):
    extra = calibrate_combine(cluster)
    rows, errs = [], []
    in_tol = signs = 0
    for h in HOLDOUTS:
        g_pred = predict_g(cluster, h, extra)
        err = g_pred - h.g_measured
        if h.role == "holdout":
            errs.append(abs(err))
            in_tol += abs(err) <= GATE_TOL
            signs += h.geom.name in NEGATIVE and g_pred < 1.0
        rows.append((h.geom.name, h.role, h.g_measured, g_pred, err))
    mae = sum(errs) / len(errs)
    ok = mae <= GATE_MAE and in_tol >= GATE_IN_TOL and signs == len(NEGATIVE)
    if verbose:
        print("Validation gate (calibration point flag back-solves combine_extra=%.3f ms/call)"
              % extra)
        print("%-8s %-12s %8s %8s %8s" % ("geom", "role", "G_meas", "G_pred", "err"))
        for name, role, gm, gp, e in rows:
            print("%-8s %-12s %8.4f %8.4f %+8.4f" % (name, role, gm, gp, e))
        print("holdout MAE=%.4f (gate 0.025)  within +-0.035: %d/6 (gate 4)  signs: %d/4 (gate 4)"
              % (mae, in_tol, signs))
        print("**%s**" % ("PASS -- extrapolation allowed" if ok
                          else "FAIL -- extrapolation forbidden; fix the model first"))
    return ok, {"mae": mae, "in_tol": int(in_tol), "signs_ok": int(signs),
                "combine_extra_ms": extra, "rows": rows}


if __name__ == "__main__":
    from .calibrate import aug_flat
    validate(aug_flat())
