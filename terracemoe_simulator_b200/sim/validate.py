"""Tier-2 gate: the model's end-to-end ``G = t(one-hop step) / t(two-hop step)`` against seven
measured training configurations.

The two-hop step is the one-hop step plus, per dispatch call, the modelled difference of the two
exchanges (the arrival chain included) and, per combine call, the same difference without the
chain plus one constant that scales with the number of (token, expert) pairs.  That constant is
solved on the ``flag`` configuration; the other six are held out and scored by
``stepgate.GateScore``.  With the shipped calibration the gate FAILS, and the tests pin that
negative result: step-level extrapolation stays locked until an overlap model explains the step
ledger.

Public surface of the reference's ``sim/validate.py`` (``HOLDOUTS`` :47-57, ``predict_g``
:60-77, ``calibrate_combine`` :80-92, ``validate`` :95-123).
"""
from __future__ import annotations

from dataclasses import dataclass

from .core import MoEGeometry, step_delta
from .records import STEP_MOE_LAYERS, STEP_RECORDS
from .stepgate import GATE_IN_TOL, GATE_MAE, GATE_TOL, GateScore

NEGATIVE = ("tok2x", "tok4x", "k8m4", "n8")
PAIRS_AT_CALIBRATION = 24576.0


@dataclass
class Holdout:
    geom: MoEGeometry
    t_off_ms: float       # measured step time of the one-hop arm
    g_measured: float
    role: str             # "calibration" | "holdout"


HOLDOUTS = [Holdout(MoEGeometry(name=name, n_groups=groups, R=R, k=k, M=M, mbs=mbs,
                                moe_layers=STEP_MOE_LAYERS), t_off, g, role)
            for name, groups, R, k, M, mbs, t_off, g, role in STEP_RECORDS]


class _CallLedger:
    """Per-call extra cost of the two-hop arm for one configuration, split by direction."""

    def __init__(self, cluster, h: Holdout):
        d = step_delta(cluster, h.geom)
        pairs = h.geom.rows_hop_b()
        self.calls = h.geom.calls_per_step_fwd() + h.geom.calls_per_step_bwd()
        self.dispatch = d["per_call_on_ms"] - d["per_call_off_ms"]
        self.combine = self.dispatch - cluster.chain_us_per_row * pairs / 1e3   # no chain back
        self.pair_scale = pairs / PAIRS_AT_CALIBRATION

    def two_hop_step(self, t_off_ms: float, combine_extra_ms: float) -> float:
        per_call = self.dispatch + self.combine + combine_extra_ms * self.pair_scale
        return t_off_ms + per_call * self.calls


def predict_g(cluster, h: Holdout, combine_extra_ms: float) -> float:
    return h.t_off_ms / _CallLedger(cluster, h).two_hop_step(h.t_off_ms, combine_extra_ms)


def calibrate_combine(cluster) -> float:
    """Per-call combine-side constant that makes the calibration configuration exact."""
    (anchor,) = [h for h in HOLDOUTS if h.role == "calibration"]
    ledger = _CallLedger(cluster, anchor)
    measured_extra = anchor.t_off_ms / anchor.g_measured - anchor.t_off_ms
    return measured_extra / ledger.calls - ledger.dispatch - ledger.combine


def validate(cluster, verbose: bool = True):
    extra = calibrate_combine(cluster)
    score, rows = GateScore(NEGATIVE), []
    for h in HOLDOUTS:
        predicted = predict_g(cluster, h, extra)
        if h.role == "holdout":
            score.add(h.geom.name, h.g_measured, predicted)
        rows.append((h.geom.name, h.role, h.g_measured, predicted, predicted - h.g_measured))
    ok = score.passed(need_signs=len(NEGATIVE))
    if verbose:
        print("\n".join(_lines(extra, rows, score, ok)))
    return ok, {"mae": score.mae, "in_tol": score.in_tol, "signs_ok": score.signs_ok,
                "combine_extra_ms": extra, "rows": rows}


def _lines(extra, rows, score, ok) -> list:
    out = ["Validation gate (calibration point flag back-solves combine_extra=%.3f ms/call)" % extra,
           "%-8s %-12s %8s %8s %8s" % ("geom", "role", "G_meas", "G_pred", "err")]
    out += ["%-8s %-12s %8.4f %8.4f %+8.4f" % row for row in rows]
    out.append("holdout MAE=%.4f (gate %.3f)  within +-%.3f: %d/6 (gate %d)  signs: %d/4 (gate 4)"
               % (score.mae, GATE_MAE, GATE_TOL, score.in_tol, GATE_IN_TOL, score.signs_ok))
    out.append("**%s**" % ("PASS -- extrapolation allowed" if ok
                           else "FAIL -- extrapolation forbidden; fix the model first"))
    return out


if __name__ == "__main__":
    from .calibrate import aug_flat
    validate(aug_flat())
