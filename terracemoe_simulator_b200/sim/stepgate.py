"""The step-level acceptance gate shared by the step validators.

A model of the end-to-end ratio ``G = t(one-hop step) / t(two-hop step)`` is accepted when, over
the held-out geometries, its mean absolute error is at most ``GATE_MAE``, at least
``GATE_IN_TOL`` predictions fall within ``GATE_TOL`` of the measurement, and every geometry known
to lose under two-hop is predicted below 1.  ``GateScore`` collects predictions and renders the
verdict; the validators differ only in how they produce a prediction.  (Reference: the gate
constants of ``sim/validate.py:41-44``.)
"""
from __future__ import annotations

GATE_MAE, GATE_TOL, GATE_IN_TOL = 0.025, 0.035, 4


class GateScore:
    def __init__(self, must_be_negative):
        self.must_be_negative = frozenset(must_be_negative)
        self.rows: list = []          # (name, measured, predicted, error), scored rows only

    def add(self, name: str, measured: float, predicted: float) -> float:
        err = predicted - measured
        self.rows.append((name, measured, predicted, err))
        return err

    @property
    def mae(self) -> float:
        return sum(abs(r[3]) for r in self.rows) / len(self.rows)

    @property
    def in_tol(self) -> int:
        return sum(1 for r in self.rows if abs(r[3]) <= GATE_TOL)

    @property
    def signs_ok(self) -> int:
        return sum(1 for name, _, pred, _ in self.rows
                   if name in self.must_be_negative and pred < 1.0)

    def n_negative(self) -> int:
        return sum(1 for r in self.rows if r[0] in self.must_be_negative)

    def passed(self, need_signs: int | None = None) -> bool:
        want = self.n_negative() if need_signs is None else need_signs
        return self.mae <= GATE_MAE and self.in_tol >= GATE_IN_TOL and self.signs_ok == want
