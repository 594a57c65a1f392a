"""Measurement records of the reference's platform A / B campaigns, as plain data.

Everything here is a number somebody measured on Ascend 910C + HCCL and published with the
reference (its ``sim/validate_sweep.py``, ``sim/twohop_measured.py``, ``sim/hostregime.py``,
``sim/hierarchy.py``, ``sim/tiers.py``, ``sim/chain_remeasured.py``).  The modules of this
package that reason about the records import them from here, so the data has one home.
B200 records are not kept in the source tree: they are produced by ``bench/sweep.py`` as JSON.
"""
from __future__ import annotations

MiB = 1 << 20

# ---- all-to-all sweeps: {world: [(total bytes per rank, median ms, pooled runs), ...]} ---------
SWEEP_A = {128: [(8 * MiB, 0.6114, 33), (16 * MiB, 0.5758, 33), (32 * MiB, 0.7072, 33),
                 (64 * MiB, 1.0162, 33), (96 * MiB, 1.3705, 33), (192 * MiB, 2.0985, 33)]}

_B_SIZES = (1 * MiB, 4 * MiB, 16 * MiB, 64 * MiB, 256 * MiB, 1024 * MiB)
SWEEP_B = {
    8: list(zip(_B_SIZES, (0.1882, 0.1613, 0.2186, 0.6039, 2.3391, 9.4678), (1,) * 6)),
    16: list(zip(_B_SIZES, (0.3089, 0.1637, 0.2394, 0.6912, 2.6408, 10.4827), (1,) * 6)),
    32: list(zip(_B_SIZES, (0.3893, 0.2269, 0.5865, 1.1790, 2.6190, 10.1870), (1,) * 6)),
    64: list(zip(_B_SIZES, (0.5376, 0.2599, 0.3601, 0.8765, 2.5861, 10.0869), (1,) * 6)),
    128: [(31457, 0.5658, 1), (62914, 0.4691, 1), (131072, 0.3933, 1), (262144, 0.4054, 1),
          (524288, 0.5148, 1), (1 * MiB, 0.4402, 2), (2 * MiB, 0.5585, 1), (4 * MiB, 0.7636, 2),
          (8 * MiB, 0.5637, 4), (16 * MiB, 0.6208, 5), (24 * MiB, 0.5971, 1),
          (25 * MiB, 0.6305, 3), (32 * MiB, 0.6958, 4), (48 * MiB, 0.8315, 1),
          (64 * MiB, 1.0672, 5), (96 * MiB, 1.3586, 1), (128 * MiB, 1.7219, 1),
          (256 * MiB, 2.7575, 2), (512 * MiB, 5.0484, 1), (1024 * MiB, 9.9033, 2)],
}

_POW2_FROM_32K = tuple(32768 << i for i in range(14))
SWEEP_C = {16: list(zip(_POW2_FROM_32K,
                        (0.1870, 0.1706, 0.1766, 0.1694, 0.1758, 0.1896, 0.1815, 0.1797, 0.1948,
                         0.2303, 0.3650, 0.6601, 1.2621, 2.4995), (6,) * 14))}
SWEEP_D = {8: list(zip(_POW2_FROM_32K[:13],
                       (0.1589, 0.1513, 0.1558, 0.1417, 0.1490, 0.1403, 0.1429, 0.1492, 0.1612,
                        0.1859, 0.3159, 0.5852, 1.1409), (12,) * 13))}


def flatten(sweep: dict) -> list:
    """{world: [(bytes, ms, runs)]} -> [(world, bytes, ms, runs)] in ascending world order."""
    return [(w, b, ms, runs) for w in sorted(sweep) for b, ms, runs in sweep[w]]

# ---- burst vs per-call all-to-all timing (ms), platform A ---------------------------------------
# sizes shared by the world-8 / world-16 host-regime tables and the supernode-boundary table
SIZES_23 = (65536, 131072, 262144, 524288, 1048576, 1572864, 2097152, 3145728, 4194304, 6291456,
            8388608, 10485760, 12582912, 16777216, 20971520, 25165824, 33554432, 50331648,
            67108864, 100663296, 134217728, 201326592, 268435456)
# per world: burst ms, per-call ms, burst spread, per-call spread (one entry per size above)
HOST_REGIME = {
    8: {"burst": (0.1278, 0.1259, 0.1202, 0.1206, 0.1179, 0.1206, 0.1217, 0.1221, 0.1248, 0.1238,
                  0.1285, 0.1131, 0.1237, 0.1599, 0.1945, 0.2283, 0.2934, 0.4275, 0.5597, 0.8273,
                  1.1109, 1.6563, 2.2259),
        "percall": (0.2378, 0.2604, 0.2403, 0.2326, 0.2418, 0.2440, 0.2498, 0.2658, 0.2699, 0.2837,
                    0.2923, 0.3326, 0.3974, 0.3954, 0.4360, 0.4284, 0.5085, 0.6389, 0.7687, 1.0491,
                    1.3283, 1.9367, 2.4922),
        "burst_spread": (0.300, 0.226, 0.066, 5.416, 0.073, 0.049, 0.037, 0.089, 0.062, 0.058,
                         1.850, 0.026, 0.006, 0.012, 0.002, 0.031, 0.003, 0.003, 0.002, 0.004,
                         0.002, 0.003, 0.004),
        "percall_spread": (0.042, 0.168, 0.051, 0.041, 0.030, 0.041, 0.050, 0.032, 0.032, 0.033,
                           0.081, 0.029, 0.149, 0.025, 0.010, 0.022, 0.062, 0.013, 0.075, 0.031,
                           0.032, 0.023, 0.027)},
    16: {"burst": (0.1339, 0.1388, 0.2304, 0.1205, 0.1207, 0.1240, 0.1212, 0.1210, 0.1296, 0.1221,
                   0.1319, 0.1561, 0.1691, 0.2057, 0.2260, 0.2627, 0.3369, 0.4868, 0.6331, 0.9331,
                   1.2290, 1.8371, 2.4633),
         "percall": (0.3128, 0.2933, 0.2878, 0.2965, 0.2903, 0.2823, 0.2805, 0.2975, 0.2950,
                     0.3293, 0.3472, 0.3784, 0.3952, 0.4416, 0.4705, 0.5210, 0.6025, 0.7163,
                     0.8495, 1.1575, 1.4744, 2.0807, 2.7017),
         "burst_spread": (0.461, 0.757, 2.986, 0.062, 0.242, 1.211, 0.207, 0.124, 6.747, 3.445,
                          0.115, 3.139, 0.019, 0.189, 0.023, 0.011, 0.007, 0.229, 0.058, 0.031,
                          0.011, 0.002, 0.011),
         "percall_spread": (0.020, 0.137, 0.016, 0.057, 0.041, 0.057, 0.020, 0.035, 0.037, 0.034,
                            0.067, 0.030, 0.035, 0.044, 0.020, 0.017, 0.011, 0.020, 0.020, 0.006,
                            0.022, 0.019, 0.041)},
}
# world 16 with the eight remote peers in the OTHER supernode: burst ms, per-call ms
ACROSS_SUPERNODE = {
    "burst": (0.2471, 0.2425, 0.2434, 0.2446, 0.2499, 0.2544, 0.2590, 0.2646, 0.2682, 0.2797,
              0.3286, 0.3782, 0.4272, 0.5275, 0.6295, 0.7295, 0.9341, 1.3302, 1.7322, 2.5314,
              3.3309, 4.9347, 6.4774),
    "percall": (0.4590, 0.4554, 0.4435, 0.4656, 0.4827, 0.4837, 0.5117, 0.5243, 0.5330, 0.6055,
                0.6574, 0.6990, 0.7609, 0.8722, 0.9603, 1.0922, 1.3069, 1.6716, 2.1005, 2.8838,
                3.6865, 5.2783, 6.8072),
}

# ---- the measured two-hop win across a supernode boundary (128 ranks, T = 4096, k = 6) ---------
# (hidden, M, q, one-hop ms, Hop A ms, chain ms, Hop B ms, splits ms)
TWOHOP_MEASURED = [(2048, 1, 6, 7.381, 1.562, 1.043, 1.477, 0.099),
                   (2048, 2, 3, 7.324, 2.646, 1.026, 1.355, 0.094),
                   (4096, 1, 6, 13.637, 2.638, 1.096, 2.270, 0.101),
                   (4096, 2, 3, 13.627, 4.813, 1.113, 2.212, 0.096)]

# ---- cross-supernode peer sweep: (peers, bytes, ms) ---------------------------------------------
PEER_SWEEP = [(n, b, ms) for b, times in (
    (67108864, (4.7749, 4.7243, 4.7307, 4.7510, 4.7711, 4.8775, 5.1810)),
    (134217728, (9.0566, 8.9636, 8.9986, 8.9874, 9.0236, 9.1272, 9.3504)),
    (268435456, (17.6363, 17.4453, 17.4877, 17.4413, 17.4614, 17.5515, 17.7128)))
    for n, ms in zip((1, 2, 4, 8, 16, 32, 64), times)]


# ---- bf16 GEMM throughput on platform A (256 samples per size) --------------------------------
# square N x N x N problems: (N, TFLOPS)
GEMM_TFLOPS = [(1024, 141.6), (2048, 271.1), (4096, 327.4), (8192, 296.7), (12288, 291.4),
               (16384, 319.2)]
# expert-FFN shapes (rows, hidden, expert width): TFLOPS
NONSQUARE_TFLOPS = {
    (1536, 2048, 5504): 309.7, (1536, 4096, 11008): 326.7, (1536, 7168, 2048): 328.3,
    (3072, 2048, 5504): 324.8, (3072, 4096, 11008): 335.9, (3072, 7168, 2048): 338.0,
    (6144, 2048, 5504): 331.4, (6144, 4096, 11008): 330.7,
}
# error of reading the square curve at the geometric mean of a non-square shape
INDEX_RULE_ERROR = {"median_abs": 0.064, "bias": -0.064, "worst": 0.109}


# ---- end-to-end steps, one-hop against two-hop (platform A, 19 MoE layers) --------------------
# (name, groups, ranks per group, k, M, micro-batches, one-hop step ms, G = t_one / t_two, role)
STEP_RECORDS = (
    ("flag", 16, 8, 6, 2, 1, 4420.4, 1.0355, "calibration"),
    ("tok2x", 16, 8, 6, 2, 2, 3343.6, 0.8845, "holdout"),
    ("tok4x", 16, 8, 6, 2, 4, 2992.7, 0.8234, "holdout"),
    ("k8m2", 16, 8, 8, 2, 1, 4791.7, 0.9935, "holdout"),
    ("k8m4", 16, 8, 8, 4, 1, 4664.9, 0.9335, "holdout"),
    ("n8", 8, 8, 6, 2, 1, 6657.5, 0.9027, "holdout"),
    ("n4", 4, 8, 6, 2, 1, 11712.0, 0.8647, "holdout"),
)
STEP_MOE_LAYERS = 19


# ---- arrival chain of platform A: instrument readings and sweeps ------------------------------
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


# ---- launch constants measured on platform A (ms) ---------------------------------------------
LAUNCH_DEVICE_INITIATED_MS = (0.036, 0.057)
LAUNCH_HOST_P2P_MS = (0.257, 0.268)
PER_CALL_DEEP_QUEUE_MS = {2: 0.087, 4: 0.098, 8: 0.129, 16: 0.134}
PER_CALL_DEEP_QUEUE_RANGE_MS = {8: (0.117, 0.133)}
PER_CALL_HOST_EXPOSED_MS = {8: 0.255, 16: 0.283}
PER_CALL_SPREAD = 0.15
HOST_SUBMIT_MS = {2: 0.039, 4: 0.043, 8: 0.058, 16: 0.076}
HOST_EXPOSURE_MS = 0.130
LAUNCH_UPPER_BOUND_MS = 0.111
