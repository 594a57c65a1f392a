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


def _best_fit(model, target, starts, lower, upper, max_nfev=40000):
    """Least squares on the RELATIVE error from several starts; keeps the start with the lowest
    median relative error.  Returns (params, median relative error)."""
    import numpy as np
    from scipy.optimize import least_squares
    best = None
    for p0 in starts:
        sol = least_squares(lambda p: (model(p) - target) / target, p0, bounds=(lower, upper),
                            max_nfev=max_nfev)
        err = float(np.median(np.abs((model(sol.x) - target) / target)))
        if best is None or err < best[1]:
            best = (sol.x, err)
    return best


def _columns(records):
    import numpy as np
    recs = _norm(records)
    world = np.array([r[1] for r in recs], dtype=float)
    size = np.array([r[2] for r in recs], dtype=float)
    ms = np.array([r[3] for r in recs], dtype=float)
    return recs, world, size, ms


def fit_frame(records, seeds=(2e4, 2e5, 2e6)) -> dict:
    """Free fit: one alpha per world plus a shared (beta_inf, x_half)."""
    import numpy as np
    recs, W, S, t = _columns(records)
    worlds = sorted({r[1] for r in recs})
    col = np.array([worlds.index(r[1]) for r in recs])
    n = len(worlds)

    def model(p):
        per_peer = S / W
        return p[:n][col] + (S * (W - 1) / W) / (p[n] * per_peer / (per_peer + p[n + 1]) * 1e6)

    p, err = _best_fit(model, t, [[0.1] * n + [110.0, s] for s in seeds],
                       [0.0] * n + [1.0, 1e2], [20.0] * n + [4000.0, 1e9])
    return {"alpha": {w: float(a) for w, a in zip(worlds, p[:n])}, "beta_inf": float(p[n]),
            "x_half": float(p[n + 1]), "median_rel_err": err, "n": len(recs)}


def fit_beta_pinned(records, alpha_of_world, seeds=(2e4, 2e5, 2e6)) -> dict:
    """Recommended fit: alpha taken from direct measurement, only (beta_inf, x_half) free."""
    import numpy as np
    recs, W, S, t = _columns(records)
    alpha = np.array([alpha_of_world(w) for w in W], dtype=float)

    def model(p):
        per_peer = S / W
        return alpha + (S * (W - 1) / W) / (p[0] * per_peer / (per_peer + p[1]) * 1e6)

    p, err = _best_fit(model, t, [[110.0, s] for s in seeds], [1.0, 1e2], [4000.0, 1e9])
    return {"beta_inf": float(p[0]), "x_half": float(p[1]), "median_rel_err": err,
            "n": len(recs)}


def fit_pinned_under_form(records, alpha_of_world, p: float = 1.0, per_peer_us=None,
                          seeds=(0.3, 1.0, 3.0)) -> dict:
    """Pinned-alpha fit of ``(alpha^p + T^p)^(1/p)`` with ``T = wire/beta_inf + (W-1)*o``;
    ``o`` (per-peer message cost, us) is fitted unless ``per_peer_us`` is given."""
    import numpy as np
    recs, W, S, t = _columns(records)
    alpha = np.array([alpha_of_world(w) for w in W], dtype=float)
    wire = S * (W - 1) / W
    fixed = per_peer_us is not None

    def model(q):
        o = per_peer_us if fixed else q[1]
        T = wire / (q[0] * 1e6) + (W - 1) * o / 1000.0
        return (alpha ** p + T ** p) ** (1.0 / p)

    starts = [[110.0] + ([] if fixed else [s]) for s in seeds]
    q, err = _best_fit(model, t, starts, [1.0] + ([] if fixed else [0.0]),
                       [4000.0] + ([] if fixed else [100.0]), max_nfev=60000)
    o = per_peer_us if fixed else float(q[1])
    return {"beta_inf": float(q[0]), "per_peer_us": o, "p": p,
            "x_half": o * float(q[0]) * 1e3 if p == 1.0 else None, "median_rel_err": err,
            "n": len(recs)}


def compare_forms(records, exponents=(1.0, 2.0, None)) -> dict:
    """Additive, quadrature, hard-max (p >= 60) and p-fitted combination forms side by side;
    alpha per world, beta_inf and the per-peer cost are free in each."""
    import numpy as np
    recs, W, S, t = _columns(records)
    worlds = sorted({r[1] for r in recs})
    col = np.array([worlds.index(r[1]) for r in recs])
    wire = S * (W - 1) / W
    n = len(worlds)

    def combine(a, T, p):
        return np.maximum(a, T) if p >= 60 else (a ** p + T ** p) ** (1.0 / p)

    out = {}
    for p in exponents:
        free_p = p is None

        def model(q, p=p, free_p=free_p):
            T = wire / (q[n] * 1e6) + (W - 1) * q[n + 1] / 1000.0
            return combine(q[:n][col], T, q[n + 2] if free_p else p)

        starts = [[0.15] * n + [110.0, s] + ([2.0] if free_p else []) for s in (0.5, 2.0, 5.0)]
        q, err = _best_fit(model, t, starts, [1e-4] * n + [1.0, 0.0] + ([0.5] if free_p else []),
                           [20.0] * n + [4000.0, 100.0] + ([60.0] if free_p else []),
                           max_nfev=60000)
        if free_p:
            label = "soft-max, p fitted"
        elif p == 1.0:
            label = "additive (shipped)"
        elif p == 2.0:
            label = "quadrature"
        elif p >= 60:
            label = "hard max"
        else:
            label = "p=%g" % p
        out[label] = {"median": err, "worst": float(np.max(np.abs((model(q) - t) / t))),
                      "beta_inf": float(q[n]), "o_us": float(q[n + 1]),
                      "p": float(q[n + 2]) if free_p else float(p),
                      "alpha": {w: float(a) for w, a in zip(worlds, q[:n])}}
    return out


def marginal_bandwidth(records, n_top: int = 4) -> dict:
    """Model-free bandwidth [GB/s]: 1 / slope of seconds against wire bytes over the ``n_top``
    largest sizes of every (frame, world).  Keys are ``world`` for frameless records."""
    series: dict = {}
    for frame, world, size, ms in _norm(records):
        series.setdefault((frame, world), []).append((size, ms))
    out = {}
    for (frame, world), pts in series.items():
        pts = sorted(pts)[-n_top:]
        if len(pts) < 2:
            continue
        xs = [s * (world - 1) / world for s, _ in pts]
        ys = [ms * 1e-3 for _, ms in pts]
        mx, my = sum(xs) / len(xs), sum(ys) / len(ys)
        den = sum((x - mx) ** 2 for x in xs)
        if den <= 0:
            continue
        slope = sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / den
        if slope > 0:
            out[(frame, world) if frame else world] = 1.0 / slope / 1e9
    return out


def audit(records, verbose: bool = True) -> dict:
    """Fit every frame on its own and print them side by side; a frame that fits far worse than
    the others points at its data, not at the model."""
    recs = _norm(records)
    results = {}
    for frame in sorted({r[0] for r in recs}):
        mine = [r for r in recs if r[0] == frame]
        if len(mine) < len({r[1] for r in mine}) + 4:
            continue
        results[frame] = fit_frame(mine)
    if verbose and results:
        print("%-12s %6s %10s %12s %10s" % ("frame", "n", "beta_inf", "x_half (KiB)", "med err"))
        for frame, r in results.items():
            print("%-12s %6d %9.1f %12.0f %9.1f%%" % (frame, r["n"], r["beta_inf"],
                                                      r["x_half"] / 1024,
                                                      r["median_rel_err"] * 100))
        seen: dict = {}
        for frame, r in results.items():
            for w in r["alpha"]:
                seen.setdefault(w, []).append(frame)
        lonely = [w for w, fs in sorted(seen.items()) if len(fs) == 1]
        if lonely:
            print("\nworlds covered by a single frame (uncheckable): %s" % lonely)
        errs = {f: r["median_rel_err"] for f, r in results.items()}
        worst = max(errs, key=errs.get)
        if errs[worst] > 2 * min(errs.values()):
            print("frame %r fits %.1fx worse than the best frame -- suspect its data first"
                  % (worst, errs[worst] / max(min(errs.values()), 1e-12)))
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
