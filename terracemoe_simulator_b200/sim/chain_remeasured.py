"""Evidence behind the arrival-chain constant of platform A.

The constant that shipped first (0.0875 us per pair) divided a 73728-pair sweep by 24576 pairs;
re-measurement puts the chain at 0.0424 us per pair in situ (1.042 ms at 24576 pairs, H = 2048)
and about 0.03 on an idle card.  This module keeps the instrument readings, the row and width
sweeps and the checks that tie them together, including the observation that the chain constant
cancels out of the step-level validation (the calibration geometry absorbs it).

Parity with the reference ``sim/chain_remeasured.py`` (:100-297).
"""
from __future__ import annotations

REFERENCE_PAIRS = 24576
REFERENCE_INPUT_ROWS = 8192
REFERENCE_H = 2048
SWEEP_INPUT_ROWS = 24576
SWEEP_QUOTA = 3
SWEEP_PAIRS = SWEEP_INPUT_ROWS * SWEEP_QUOTA
# (when, histogram primitive, chain ms at the reference point)
CALIBRATION_INSTRUMENT = [("2026-08-23 00:41", "bincount", 1.1924),
                          ("2026-08-23 01:01", "bincount", 1.1811),
                          ("2026-08-23 08:11", "fixed_hist", 0.7810),
                          ("2026-08-23 12:21", "fixed_hist", 0.7721),
                          ("2026-08-24 07:06", "fixed_hist", 0.7758)]
HISTOGRAM_CHANGE = (0.7939, 0.3270)       # histogram step alone: bincount ms -> fixed_hist ms
# (input rows, pairs, ms on node 14, ms on node 15)
AUGUST_ROW_SWEEP = [(1024, 3072, 0.2418, 0.2541), (2048, 6144, 0.2812, 0.2808),
                    (4096, 12288, 0.4300, 0.4210), (8192, 24576, 0.7446, 0.7295),
                    (16384, 49152, 1.4368, 1.3963), (24576, 73728, 2.5573, 2.4464),
                    (32768, 98304, 3.2951, 3.3382), (49152, 147456, 4.9724, 4.9216),
                    (65536, 196608, 6.5339, 6.4078)]
AUGUST_WIDTH_SWEEP = [(1024, 2.3586, 2.3781), (2048, 2.5521, 2.4672), (4096, 2.8834, 2.8165),
                      (8192, 3.8183, 3.7550)]
ROW_SWEEP = [(1024, 0.3420), (2048, 0.3562), (4096, 0.3889), (8192, 0.4482), (12288, 0.4984),
             (16384, 0.5809), (24576, 0.7150), (32768, 0.8494), (49152, 1.1942), (65536, 1.7768)]
WIDTH_SWEEP = [(1024, 0.7168), (2048, 0.7235), (4096, 0.7739), (8192, 1.0025)]
# (pairs, H, reference chain ms, live chain ms)
LIVE_VS_REFERENCE = [(8192, 2048, 0.4685, 0.4900), (8192, 8192, 0.4854, 0.5156),
                     (24576, 2048, 0.6855, 0.7752), (24576, 8192, 0.9955, 1.0520),
                     (65536, 2048, 1.7767, 2.0674), (65536, 8192, 2.7319, 3.0258)]
REFERENCE_READINGS = [("2026-08-23 instrument", 0.7810), ("2026-08-23 instrument", 0.7721),
                      ("2026-08-24 instrument", 0.7758), ("2026-08-26 sweep, node 14", 0.7446),
                      ("2026-08-26 sweep, node 15", 0.7295), ("2026-09-08 re-measurement", 0.7150)]
PRE_CORRECTION_LEVEL_MS = 2.15
US_PER_ROW = {"shipped before 2026-09-08": 0.0875, "one idle card, August": 0.0303,
              "one idle card, September": 0.0291, "in situ, 8 cards (shipped)": 0.0424,
              "fused design target": 0.0120}


def us_per_row_here(pairs: int = REFERENCE_PAIRS) -> float:
    return dict(ROW_SWEEP)[pairs] * 1000.0 / pairs


def live_overhead() -> tuple:
    ratios = [live / ref for _p, _h, ref, live in LIVE_VS_REFERENCE]
    return min(ratios), max(ratios)


def august_width_means() -> dict:
    return {H: (a + b) / 2.0 for H, a, b in AUGUST_WIDTH_SWEEP}


def published_sweep_is_at_pairs() -> bool:
    """The published width table equals the two-node mean of the 73728-pair sweep."""
    from .machine import CHAIN_H_SWEEP_MS
    return all(abs(CHAIN_H_SWEEP_MS[H] - m) < 0.005 for H, m in august_width_means().items())


def ratio_to_calibration() -> dict:
    from .machine import CHAIN_H_SWEEP_MS
    return {H: (CHAIN_H_SWEEP_MS[H] / SWEEP_PAIRS) / (ms / REFERENCE_PAIRS)
            for H, ms in WIDTH_SWEEP}


def reference_spread() -> tuple:
    vals = [ms for _, ms in REFERENCE_READINGS]
    return min(vals), max(vals)


def overcharge() -> float:
    vals = sorted(ms for _, ms in REFERENCE_READINGS)
    median = (vals[len(vals) // 2 - 1] + vals[len(vals) // 2]) / 2.0
    return PRE_CORRECTION_LEVEL_MS / median


def histogram_speedup() -> float:
    return HISTOGRAM_CHANGE[0] / HISTOGRAM_CHANGE[1]


def chain_cancels_in_validation(values=(0.0875, 0.0424, 0.0303, 0.0)) -> dict:
    """{chain constant: (holdout MAE of the step-level gate, predicted G per geometry)}: the
    MAE does not move with the constant because the calibration geometry absorbs it."""
    import dataclasses
    from .calibrate import flat_supernode
    from .validate import HOLDOUTS, calibrate_combine, predict_g
    base = flat_supernode()
    out = {}
    for v in values:
        c = dataclasses.replace(base, chain_us_per_row=v)
        extra = calibrate_combine(c)
        gs = tuple(predict_g(c, h, extra) for h in HOLDOUTS)
        errs = [abs(g - h.g_measured) for g, h in zip(gs, HOLDOUTS) if h.role == "holdout"]
        out[v] = (sum(errs) / len(errs), gs)
    return out


def breakevens() -> dict:
    from .uncertainty import breakeven_ratio
    return {k: breakeven_ratio(v) for k, v in US_PER_ROW.items()}


def main() -> None:
    print("The width sweep ran %d input rows at quota %d = %d pairs; the calibration point is "
          "%d pairs." % (SWEEP_INPUT_ROWS, SWEEP_QUOTA, SWEEP_PAIRS, REFERENCE_PAIRS))
    print("published width table is the 73728-pair sweep: %s" % published_sweep_is_at_pairs())
    print("readings at %d pairs, H = %d:" % (REFERENCE_PAIRS, REFERENCE_H))
    for label, ms in REFERENCE_READINGS:
        print("   %-28s %.4f ms" % (label, ms))
    lo, hi = reference_spread()
    print("spread %.1f%%; the pre-correction level %.2f ms overcharged by %.2fx"
          % (100 * (hi - lo) / lo, PRE_CORRECTION_LEVEL_MS, overcharge()))
    print("fixed-length histogram instead of bincount: %.2fx on that step" % histogram_speedup())
    print("live chain against the reference chain: %.2fx - %.2fx" % live_overhead())
    print("us per pair, and the breakeven hierarchy ratio each implies:")
    be = breakevens()
    for k, v in US_PER_ROW.items():
        print("   %-30s %.4f   breakeven %.2f" % (k, v, be[k]))
    print("step-level validation MAE by chain constant (it cancels):")
    for v, (mae, _) in chain_cancels_in_validation().items():
        print("   %.4f -> MAE %.4f" % (v, mae))


if __name__ == "__main__":
    main()
