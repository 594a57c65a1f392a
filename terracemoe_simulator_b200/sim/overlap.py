"""Six one-parameter overlap hypotheses, fitted on the calibration configuration and scored on
the six holdouts of the step-level gate.

Every hypothesis says the same kind of thing: of the modelled step difference ``d_model``
(two-hop minus one-hop, nothing overlapped) a part is hidden behind compute, and that part is
proportional to some quantity of the step -- the difference itself, the number of calls, the
fixed per-call overhead, the compute time, or the difference per micro-batch:

    d_predicted = d_model - c * basis(step)

The coefficient ``c`` is solved on the calibration configuration, then reported in the
parametrisation each family is known by (e.g. ``phi = 1 - c`` for the proportional family).
All six fail the gate -- a pinned negative result: no single scalar of "how much communication
hides behind compute" explains the measured step differences.

Public surface of the reference's ``sim/overlap.py`` (``decompose`` :60-86, families :99-129,
``evaluate`` :132-165).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .core import step_delta
from .stepgate import GATE_IN_TOL, GATE_MAE, GATE_TOL, GateScore  # noqa: F401  (re-exported)
from .validate import HOLDOUTS

NEG_NAMES = {"tok2x", "tok4x", "k8m4", "n8", "n4"}


@dataclass(frozen=True)
class Decomp:
    """What is known about one measured configuration: the measurement (``g_meas``, ``t_off``),
    its shape (``calls``, ``mbs``) and the model's view of it, all in ms per step."""
    name: str
    role: str
    g_meas: float
    t_off: float        # measured one-hop step
    calls: int
    mbs: int
    d_model: float      # modelled step difference (two-hop minus one-hop)
    fixed: float        # the part of d_model that is arrival chain + splits read-back
    comm_off: float     # modelled communication of the one-hop arm

    @property
    def d_meas(self) -> float:          # measured step difference
        return self.t_off * (1.0 / self.g_meas - 1.0)

    @property
    def t_comp(self) -> float:          # one-hop step minus its communication
        return self.t_off - self.comm_off

    def g_from_delta(self, delta_ms: float) -> float:
        return self.t_off / (self.t_off + delta_ms)


def _decompose_one(cluster, h) -> Decomp:
    priced, geom = step_delta(cluster, h.geom), h.geom
    calls = priced["calls_per_step"]
    overhead = cluster.splits_sync_ms + cluster.chain_us_per_row * geom.rows_hop_b() / 1e3
    return Decomp(geom.name, h.role, h.g_measured, h.t_off_ms, calls, geom.mbs,
                  priced["step_delta_ms"], calls * overhead, calls * priced["per_call_off_ms"])


def decompose(cluster) -> list:
    return [_decompose_one(cluster, h) for h in HOLDOUTS]


@dataclass(frozen=True)
class Family:
    """``d = d_model - c * basis``; ``shown(c)`` is the parameter the family reports."""
    key: str
    desc: str
    n_params: int
    basis: Callable
    shown: Callable = staticmethod(lambda c: c)

    def coefficient(self, cal: Decomp) -> float:
        b = self.basis(cal)
        return (cal.d_model - cal.d_meas) / b if b else 0.0

    def delta(self, d: Decomp, c: float) -> float:
        return d.d_model - c * self.basis(d)


FAMILIES = (
    Family("M0", "naive: d = d_model (no overlap)", 0, lambda d: 0.0),
    Family("M1", "prop: d = phi*d_model", 1, lambda d: d.d_model, lambda c: 1.0 - c),
    Family("M2", "hide/call: d = d_model-h*calls", 1, lambda d: float(d.calls)),
    Family("M3", "hide-fixed: d = d_model-phi*fixed", 1, lambda d: d.fixed),
    Family("M4", "hide~comp: d = d_model-c*T_comp", 1, lambda d: d.t_comp),
    Family("M5", "expose-mb: d = d_model*(1-lam/mbs)", 1, lambda d: d.d_model / d.mbs),
)


def _families() -> list:
    return list(FAMILIES)


def _score(fam: Family, cal: Decomp, holdouts) -> dict:
    c = fam.coefficient(cal)
    score = GateScore(NEG_NAMES)
    for d in holdouts:
        score.add(d.name, d.g_meas, d.g_from_delta(fam.delta(d, c)))
    return {"param": fam.shown(c) if fam.n_params else 0.0, "mae": score.mae,
            "in_tol": score.in_tol, "signs_ok": score.signs_ok, "n_neg": score.n_negative(),
            "rows": list(score.rows), "desc": fam.desc, "gate": score.passed()}


def evaluate(cluster, verbose: bool = True) -> dict:
    parts = decompose(cluster)
    by_role = {role: [d for d in parts if d.role == role] for role in ("calibration", "holdout")}
    (cal,) = by_role["calibration"]
    results = {fam.key: _score(fam, cal, by_role["holdout"]) for fam in FAMILIES}
    if verbose:
        print("\n".join(_report(parts, results)))
    return results


def _report(parts, results) -> list:
    out = ["%-7s %4s %8s %11s %11s %9s %8s" % ("geom", "mbs", "G_meas", "d_meas_ms", "d_model_ms",
                                               "fixed", "expose")]
    out += ["%-7s %4d %8.4f %11.1f %11.1f %9.1f %8.3f"
            % (d.name, d.mbs, d.g_meas, d.d_meas, d.d_model, d.fixed, d.d_meas / d.d_model)
            for d in parts]
    out += ["", "%-4s %-36s %9s %7s %8s %6s %5s" % ("fam", "structure", "param", "MAE", "+-0.035",
                                                   "signs", "gate")]
    out += ["%-4s %-36s %9.4f %7.4f %6d/6 %4d/%d %5s"
            % (key, r["desc"], r["param"], r["mae"], r["in_tol"], r["signs_ok"], r["n_neg"],
               "PASS" if r["gate"] else "FAIL") for key, r in results.items()]
    winners = ", ".join(key for key, r in results.items() if r["gate"])
    out.append("families passing the gate: %s"
               % (winners or "none -- no one-parameter overlap explains the steps"))
    return out


if __name__ == "__main__":
    from .calibrate import flat_supernode
    evaluate(flat_supernode())
