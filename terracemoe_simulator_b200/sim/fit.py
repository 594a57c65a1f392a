"""Fit the alpha/beta model to measured all-to-all (or fused dispatch) sweeps.

Record schema: ``{"frame": str, "world": int, "bytes": float, "ms": float}`` -- ``bytes`` is the
total payload one rank sends in one exchange (all peers, self share included), ``ms`` the
device-timed duration, max over ranks.  A frame groups records that share one measurement
protocol; frames are fitted separately and then compared (``audit``).

    predicted ms = alpha(world) + bytes*(world-1)/world / (beta_eff(bytes/world) * 1e6)
    beta_eff(x)  = beta_inf * x / (x + x_half)

Fitting alpha, beta_inf and x_half together is degenerate (a larger x_half trades against a
smaller alpha), so the recommended route is ``fit_beta_pinned``: measure alpha directly (tiny
messages) and fit only ``(beta_inf, x_half)``.  ``marginal_bandwidth`` is the model-free check:
the slope of time against wire bytes over the largest sizes.

Parity with the reference ``sim/fit.py``: ``load_records`` :92, ``beta_eff``/``predict_ms``
:103-114, ``fit_frame`` :117, ``fit_beta_pinned`` :157, ``fit_pinned_under_form`` :188,
``compare_forms`` :244, ``marginal_bandwidth`` :323, ``audit`` :374, ``_demo`` :415.
scipy is imported lazily: only the fitting entry points need it.
"""
from __future__ import annotations

import json
import math

BETA_INF_GBPS = 118.0
X_HALF_BYTES = 320 * 1024


def _norm(records) -> list:
    """Accept dict records, (frame, world, bytes, ms) tuples or (world, bytes, ms) triples."""
    out = []
    for r in records:
        if isinstance(r, dict):
            out.append((str(r.get("frame", "default")), int(r["world"]), float(r["bytes"]),
                        float(r["ms"])))
        elif len(r) == 3:
            out.append(("", int(r[0]), float(r[1]), float(r[2])))
        else:
            out.append((str(r[0]), int(r[1]), float(r[2]), float(r[3])))
    return out


def load_records(path: str) -> list:
    with open(path, encoding="utf-8") as fh:
        raw = json.load(fh)
    if isinstance(raw, dict):
        raw = raw.get("records", [])
    return [r for r in _norm(raw) if r[3] > 0 and r[1] >= 2 and r[2] > 0]


def beta_eff(per_peer_bytes: float, beta_inf: float = BETA_INF_GBPS,
             x_half: float = X_HALF_BYTES) -> float:
    x = max(float(per_peer_bytes), 0.0)
    return beta_inf * x / (x + x_half)


def predict_ms(world: int, total_bytes: float, alpha_ms: float,
               beta_inf: float = BETA_INF_GBPS, x_half: float = X_HALF_BYTES) -> float:
    wire = total_bytes * (world - 1) / world
    return alpha_ms + wire / (beta_eff(total_bytes / world, beta_inf, x_half) * 1e6)


class _Sweep:
    """Column view of a record list (numpy arrays): ``world``, ``size`` (bytes per rank),
    ``ms``, plus the derived ``wire`` bytes, ``per_peer`` message size and, per record, the index
    of its world among the distinct ``worlds``."""

    def __init__(self, records):
        import numpy as np
        self.records = _norm(records)
        cols = list(zip(*[(r[1], r[2], r[3]) for r in self.records])) or [(), (), ()]
        self.world, self.size, self.ms = (np.asarray(c, dtype=float) for c in cols)
        self.wire = self.size * (self.world - 1.0) / self.world
        self.per_peer = self.size / self.world
        self.worlds = sorted({r[1] for r in self.records})
        self.slot = np.asarray([self.worlds.index(r[1]) for r in self.records], dtype=int)

    def __len__(self) -> int:
        return len(self.records)

    def pinned_alpha(self, alpha_of_world):
        import numpy as np
        return np.asarray([alpha_of_world(w) for w in self.world], dtype=float)

    def saturating_ms(self, beta_inf, x_half):
        """wire / beta_eff(per-peer size), in ms."""
        return self.wire * (self.per_peer + x_half) / (1e6 * beta_inf * self.per_peer)

    def per_message_ms(self, beta_inf, per_peer_us):
        """wire / beta_inf plus an explicit cost per peer message, in ms."""
        return self.wire / (1e6 * beta_inf) + 1e-3 * per_peer_us * (self.world - 1.0)


class _Params:
    """Named blocks of one flat parameter vector with their bounds and start values."""

    def __init__(self):
        self.names, self.sizes, self.low, self.high = [], [], [], []

    def block(self, name: str, size: int, low: float, high: float) -> "_Params":
        self.names.append(name)
        self.sizes.append(size)
        self.low += [low] * size
        self.high += [high] * size
        return self

    def split(self, vector) -> dict:
        out, at = {}, 0
        for name, size in zip(self.names, self.sizes):
            out[name] = vector[at:at + size] if size != 1 else vector[at]
            at += size
        return out

    def starts(self, **values) -> list:
        """One start vector; a scalar value fills its block."""
        vec = []
        for name, size in zip(self.names, self.sizes):
            vec += [float(values[name])] * size
        return vec


def _best_fit(model, target, starts, lower, upper, max_nfev=40000):
    """Least squares on the RELATIVE error from several starts; keeps the start with the lowest
    median relative error.  Returns (params, median relative error)."""
    import numpy as np
    from scipy.optimize import least_squares

    def relative(p):
        return model(p) / target - 1.0
    runs = [least_squares(relative, p0, bounds=(lower, upper), max_nfev=max_nfev).x
            for p0 in starts]
    scored = [(float(np.median(np.abs(relative(x)))), i) for i, x in enumerate(runs)]
    err, winner = min(scored)
    return runs[winner], err


def _solve(layout: _Params, model_of, sweep: _Sweep, starts, max_nfev=40000):
    """Fit ``model_of(named blocks)`` to the sweep; returns (named blocks, median error, model)."""
    def model(vector):
        return model_of(layout.split(vector))
    best, err = _best_fit(model, sweep.ms, starts, layout.low, layout.high, max_nfev)
    return layout.split(best), err, model(best)


def _alpha_table(sweep: _Sweep, alphas) -> dict:
    return {w: float(a) for w, a in zip(sweep.worlds, alphas)}


def fit_frame(records, seeds=(2e4, 2e5, 2e6)) -> dict:
    """Free fit: one alpha per world plus a shared (beta_inf, x_half)."""
    sweep = _Sweep(records)
    layout = (_Params().block("alpha", len(sweep.worlds), 0.0, 20.0)
              .block("beta_inf", 1, 1.0, 4000.0).block("x_half", 1, 1e2, 1e9))
    import numpy as np
    got, err, _ = _solve(
        layout, lambda v: np.atleast_1d(v["alpha"])[sweep.slot]
        + sweep.saturating_ms(v["beta_inf"], v["x_half"]), sweep,
        [layout.starts(alpha=0.1, beta_inf=110.0, x_half=seed) for seed in seeds])
    return {"alpha": _alpha_table(sweep, np.atleast_1d(got["alpha"])),
            "beta_inf": float(got["beta_inf"]), "x_half": float(got["x_half"]),
            "median_rel_err": err, "n": len(sweep)}


def fit_beta_pinned(records, alpha_of_world, seeds=(2e4, 2e5, 2e6)) -> dict:
    """Recommended fit: alpha taken from direct measurement, only (beta_inf, x_half) free."""
    sweep = _Sweep(records)
    alpha = sweep.pinned_alpha(alpha_of_world)
    layout = _Params().block("beta_inf", 1, 1.0, 4000.0).block("x_half", 1, 1e2, 1e9)
    got, err, _ = _solve(layout,
                         lambda v: alpha + sweep.saturating_ms(v["beta_inf"], v["x_half"]), sweep,
                         [layout.starts(beta_inf=110.0, x_half=seed) for seed in seeds])
    return {"beta_inf": float(got["beta_inf"]), "x_half": float(got["x_half"]),
            "median_rel_err": err, "n": len(sweep)}


def _soft_combine(fixed, transfer, p):
    """(fixed^p + transfer^p)^(1/p); from p = 60 on the hard maximum."""
    import numpy as np
    if p >= 60:
        return np.maximum(fixed, transfer)
    return (fixed ** p + transfer ** p) ** (1.0 / p)


def fit_pinned_under_form(records, alpha_of_world, p: float = 1.0, per_peer_us=None,
                          seeds=(0.3, 1.0, 3.0)) -> dict:
    """Pinned-alpha fit of ``(alpha^p + T^p)^(1/p)`` with ``T = wire/beta_inf + (W-1)*o``;
    ``o`` (per-peer message cost, us) is fitted unless ``per_peer_us`` is given."""
    sweep = _Sweep(records)
    alpha = sweep.pinned_alpha(alpha_of_world)
    layout = _Params().block("beta_inf", 1, 1.0, 4000.0)
    if per_peer_us is None:
        layout.block("o", 1, 0.0, 100.0)
        starts = [layout.starts(beta_inf=110.0, o=seed) for seed in seeds]
    else:
        starts = [layout.starts(beta_inf=110.0) for _ in seeds]

    def model(v):
        cost = v["o"] if per_peer_us is None else per_peer_us
        return (alpha ** p + sweep.per_message_ms(v["beta_inf"], cost) ** p) ** (1.0 / p)

    got, err, _ = _solve(layout, model, sweep, starts, max_nfev=60000)
    cost = float(got["o"]) if per_peer_us is None else per_peer_us
    beta = float(got["beta_inf"])
    return {"beta_inf": beta, "per_peer_us": cost, "p": p,
            "x_half": 1e3 * beta * cost if p == 1.0 else None, "median_rel_err": err,
            "n": len(sweep)}


def _form_label(p) -> str:
    if p is None:
        return "soft-max, p fitted"
    fixed = {1.0: "additive (shipped)", 2.0: "quadrature"}
    if p in fixed:
        return fixed[p]
    return "hard max" if p >= 60 else "p=%g" % p


def compare_forms(records, exponents=(1.0, 2.0, None)) -> dict:
    """Additive, quadrature, hard-max (p >= 60) and p-fitted combination forms side by side;
    alpha per world, beta_inf and the per-peer cost are free in each."""
    import numpy as np
    sweep = _Sweep(records)
    table = {}
    for p in exponents:
        layout = (_Params().block("alpha", len(sweep.worlds), 1e-4, 20.0)
                  .block("beta_inf", 1, 1.0, 4000.0).block("o", 1, 0.0, 100.0))
        seed_values = dict(alpha=0.15, beta_inf=110.0)
        if p is None:
            layout.block("p", 1, 0.5, 60.0)
            seed_values["p"] = 2.0

        def model(v, p=p):
            alphas = np.atleast_1d(v["alpha"])[sweep.slot]
            return _soft_combine(alphas, sweep.per_message_ms(v["beta_inf"], v["o"]),
                                 v["p"] if p is None else p)

        got, err, fitted = _solve(layout, model, sweep,
                                  [layout.starts(o=o, **seed_values) for o in (0.5, 2.0, 5.0)],
                                  max_nfev=60000)
        table[_form_label(p)] = {
            "median": err, "worst": float(np.max(np.abs(fitted / sweep.ms - 1.0))),
            "beta_inf": float(got["beta_inf"]), "o_us": float(got["o"]),
            "p": float(got["p"] if p is None else p),
            "alpha": _alpha_table(sweep, np.atleast_1d(got["alpha"]))}
    return table


def marginal_bandwidth(records, n_top: int = 4) -> dict:
    """Model-free bandwidth [GB/s]: 1 / slope of seconds against wire bytes over the ``n_top``
    largest sizes of every (frame, world).  Keys are ``world`` for frameless records."""
    by_series: dict = {}
    for frame, world, size, ms in _norm(records):
        by_series.setdefault((frame, world), []).append((size * (world - 1) / world, 1e-3 * ms))
    rates = {}
    for (frame, world), points in by_series.items():
        top = sorted(points)[-n_top:]
        n = len(top)
        if n < 2:
            continue
        sx, sy = sum(x for x, _ in top), sum(y for _, y in top)
        sxx, sxy = sum(x * x for x, _ in top), sum(x * y for x, y in top)
        spread = n * sxx - sx * sx
        slope = (n * sxy - sx * sy) / spread if spread > 0 else 0.0
        if slope > 0:
            rates[(frame, world) if frame else world] = 1e-9 / slope
    return rates


def audit(records, verbose: bool = True) -> dict:
    """Fit every frame on its own and print them side by side; a frame that fits far worse than
    the others points at its data, not at the model."""
    by_frame: dict = {}
    for rec in _norm(records):
        by_frame.setdefault(rec[0], []).append(rec)
    results = {}
    for frame in sorted(by_frame):
        mine = by_frame[frame]
        enough = len(mine) >= 4 + len({r[1] for r in mine})       # parameters + a few spare
        if enough:
            results[frame] = fit_frame(mine)
    if verbose and results:
        from ._text import Column, render_table
        cols = [Column("frame", "%-12s", lambda kv: kv[0]), Column("n", "%6d", lambda kv: kv[1]["n"]),
                Column("beta_inf", "%10.1f", lambda kv: kv[1]["beta_inf"]),
                Column("x_half (KiB)", "%12.0f", lambda kv: kv[1]["x_half"] / 1024),
                Column("med err", "%10s", lambda kv: "%.1f%%" % (100 * kv[1]["median_rel_err"]))]
        header, _rule, *body = render_table(cols, results.items())
        print("\n".join([header, *body]))
        covered: dict = {}
        for frame, res in results.items():
            for w in res["alpha"]:
                covered.setdefault(w, set()).add(frame)
        lonely = sorted(w for w, frames in covered.items() if len(frames) == 1)
        if lonely:
            print("\nworlds covered by a single frame (uncheckable): %s" % lonely)
        errs = {frame: res["median_rel_err"] for frame, res in results.items()}
        worst, best = max(errs, key=errs.get), min(errs.values())
        if errs[worst] > 2 * best:
            print("frame %r fits %.1fx worse than the best frame -- suspect its data first"
                  % (worst, errs[worst] / max(best, 1e-12)))
    return results


def _demo() -> None:
    """Self-check on synthetic data: the free fit reproduces the times but not x_half (the
    degeneracy), the pinned fit recovers both constants."""
    alpha, binf, xh = 0.30, 118.0, 320 * 1024
    recs = [("synthetic", w, float(s), predict_ms(w, s, alpha, binf, xh))
            for s in (2 ** 20, 4 * 2 ** 20, 16 * 2 ** 20, 64 * 2 ** 20, 256 * 2 ** 20)
            for w in (8, 16, 128)]
    free = fit_frame(recs)
    print("free alpha : beta_inf %.1f (truth %.1f), x_half %.0f KiB (truth %.0f), err %.2g%%"
          % (free["beta_inf"], binf, free["x_half"] / 1024, xh / 1024,
             free["median_rel_err"] * 100))
    pinned = fit_beta_pinned(recs, lambda _w: alpha)
    print("pinned alpha: beta_inf %.1f, x_half %.0f KiB, err %.2g%%"
          % (pinned["beta_inf"], pinned["x_half"] / 1024, pinned["median_rel_err"] * 100))
    assert math.isclose(free["beta_inf"], binf, rel_tol=0.02)
    assert math.isclose(pinned["x_half"], xh, rel_tol=0.05)


if __name__ == "__main__":
    _demo()
