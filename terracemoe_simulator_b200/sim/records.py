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
