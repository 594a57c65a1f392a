"""Evidence behind the arrival-chain constant of platform A.

The constant that shipped first (0.0875 us per pair) divided the time of a 73728-pair sweep by
24576 pairs; re-measurement puts the chain at 0.0424 us per pair in situ (1.042 ms at 24576
pairs, H = 2048) and about 0.03 on an idle card.  The readings themselves live in
``sim/records.py``; this module asks the questions that tie them together: is the published
width table the 73728-pair sweep, how far do the repeated readings of the reference point
spread, by how much did the first constant overcharge, what did the fixed-length histogram buy,
what does each candidate constant imply for the breakeven hierarchy ratio -- and it shows that
the constant cancels out of the step-level validation, because the calibration configuration
absorbs it.

Public surface of the reference's ``sim/chain_remeasured.py`` (:100-297).
"""
from __future__ import annotations

import dataclasses
import statistics

from .records import (AUGUST_ROW_SWEEP, AUGUST_WIDTH_SWEEP, CALIBRATION_INSTRUMENT,  # noqa: F401
                      HISTOGRAM_CHANGE, LIVE_VS_REFERENCE, PRE_CORRECTION_LEVEL_MS,
                      REFERENCE_H, REFERENCE_INPUT_ROWS, REFERENCE_PAIRS, REFERENCE_READINGS,
                      ROW_SWEEP, SWEEP_INPUT_ROWS, SWEEP_PAIRS, SWEEP_QUOTA, US_PER_ROW,
                      WIDTH_SWEEP)


def _reference_ms() -> list:
    return [ms for _label, ms in REFERENCE_READINGS]


def us_per_row_here(pairs: int = REFERENCE_PAIRS) -> float:
    """Chain cost per pair, in us, of the September row sweep at ``pairs`` pairs."""
    (ms,) = [t for n, t in ROW_SWEEP if n == pairs]
    return 1e3 * ms / pairs


def live_overhead() -> tuple:
    """(smallest, largest) ratio of the live chain's time to the reference chain's."""
    ratios = sorted(row[3] / row[2] for row in LIVE_VS_REFERENCE)
    return ratios[0], ratios[-1]


def august_width_means() -> dict:
    return {width: statistics.fmean(nodes) for width, *nodes in AUGUST_WIDTH_SWEEP}


def published_sweep_is_at_pairs() -> bool:
    """The published width table equals the two-node mean of the 73728-pair sweep."""
    from .machine import CHAIN_H_SWEEP_MS
    gaps = (abs(CHAIN_H_SWEEP_MS[w] - mean) for w, mean in august_width_means().items())
    return max(gaps) < 0.005


def ratio_to_calibration() -> dict:
    """Per hidden width: cost per pair of the published (73728-pair) table over the cost per
    pair measured at the calibration point."""
    from .machine import CHAIN_H_SWEEP_MS
    return {w: (CHAIN_H_SWEEP_MS[w] / SWEEP_PAIRS) * REFERENCE_PAIRS / ms for w, ms in WIDTH_SWEEP}


def reference_spread() -> tuple:
    readings = _reference_ms()
    return min(readings), max(readings)


def overcharge() -> float:
    return PRE_CORRECTION_LEVEL_MS / statistics.median(_reference_ms())


def histogram_speedup() -> float:
    before, after = HISTOGRAM_CHANGE
    return before / after


def chain_cancels_in_validation(values=(0.0875, 0.0424, 0.0303, 0.0)) -> dict:
    """{chain constant: (holdout MAE of the step-level gate, predicted G per configuration)}: the
    MAE does not move with the constant because the calibration configuration absorbs it."""
    from .calibrate import flat_supernode
    from .validate import HOLDOUTS, calibrate_combine, predict_g
    base, held = flat_supernode(), [h.role == "holdout" for h in HOLDOUTS]

    def outcome(us_per_row: float):
        cluster = dataclasses.replace(base, chain_us_per_row=us_per_row)
        extra = calibrate_combine(cluster)
        predicted = tuple(predict_g(cluster, h, extra) for h in HOLDOUTS)
        misses = [abs(g - h.g_measured) for g, h, use in zip(predicted, HOLDOUTS, held) if use]
        return statistics.fmean(misses), predicted

    return {v: outcome(v) for v in values}


def breakevens() -> dict:
    from .uncertainty import breakeven_ratio
    return {label: breakeven_ratio(us) for label, us in US_PER_ROW.items()}


def report() -> list:
    lo, hi = reference_spread()
    implied = breakevens()
    out = ["The width sweep ran %d input rows at quota %d = %d pairs; the calibration point is %d "
           "pairs." % (SWEEP_INPUT_ROWS, SWEEP_QUOTA, SWEEP_PAIRS, REFERENCE_PAIRS),
           "published width table is the 73728-pair sweep: %s" % published_sweep_is_at_pairs(),
           "readings at %d pairs, H = %d:" % (REFERENCE_PAIRS, REFERENCE_H)]
    out += ["   %-28s %.4f ms" % reading for reading in REFERENCE_READINGS]
    out += ["spread %.1f%%; the pre-correction level %.2f ms overcharged by %.2fx"
            % (100 * (hi / lo - 1.0), PRE_CORRECTION_LEVEL_MS, overcharge()),
            "fixed-length histogram instead of bincount: %.2fx on that step" % histogram_speedup(),
            "live chain against the reference chain: %.2fx - %.2fx" % live_overhead(),
            "us per pair, and the breakeven hierarchy ratio each implies:"]
    out += ["   %-30s %.4f   breakeven %.2f" % (label, us, implied[label])
            for label, us in US_PER_ROW.items()]
    out.append("step-level validation MAE by chain constant (it cancels):")
    out += ["   %.4f -> MAE %.4f" % (us, mae)
            for us, (mae, _g) in chain_cancels_in_validation().items()]
    return out


def main() -> None:
    print("\n".join(report()))


if __name__ == "__main__":
    main()
