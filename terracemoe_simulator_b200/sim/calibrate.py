"""Calibration constants and cluster builders.

Two families of constants live here:
  * platform "A" (Ascend 910C + HCCL), the numbers the reference distilled from its measurement
    campaigns (``sim/calibrate.py:58-270`` of the reference) -- kept so that every published
    table and gate of the cost model can be reproduced;
  * platform "B200" (8 x B200, one NVSwitch domain, fused peer-memory transport), fitted from
    the sweep this repository's ``bench/sweep.py`` writes (``b200_from_records``), with defaults
    from the first measurements on that machine.

Builders: ``saturating_beta`` (beta(x) = beta_inf * x / (x + x_half), i.e. a fixed cost
x_half / beta_inf per peer message), ``flat_supernode``, ``second_machine``,
``supernode_under_form``, ``synthetic(ratio)``, ``b200_nvswitch``.
"""
from __future__ import annotations

from .core import ClusterSpec, Level

# ---- platform A -------------------------------------------------------------------------------
ALPHA_PTS = [(2, 0.09), (8, 0.111), (16, 0.157), (128, 0.378), (256, 0.735), (512, 1.859)]
ALPHA_REGIME = "deep queue (host runs ahead)"
ALPHA_BY_REGIME = {"deep queue": {8: 0.114, 16: 0.120}, "host exposed": {8: 0.229, 16: 0.261}}
ALPHA_CORPUS_JOINT_FIT = {"C": {"world": 16, "alpha": 0.157, "beta_inf": 131.8},
                          "D": {"world": 8, "alpha": 0.119, "beta_inf": 152.7}}
PHYSICAL_CEILING_GBPS = 122.4
BETA_FLAT = 117.8
X_HALF_FLAT = 54 * 1024
X_HALF_CI = (30 * 1024, 87 * 1024)
X_HALF_GATE_UPPER = 77 * 1024
PER_PEER_MESSAGE_US = X_HALF_FLAT / (BETA_FLAT * 1e9) * 1e6
MARGINAL_BW_BY_WORLD = {8: 107.4, 16: 103.0, 128: 120.6}
MARGINAL_BW_SECOND_MACHINE = {8: 99.6, 16: 96.5, 32: 106.9, 64: 107.1, 128: 113.3}
BETA_FAST = 122.4
CROSS_NODE_RATIO = 0.974
SPLITS_SYNC_MS = 0.044
CHAIN_US_PER_ROW = 1.042 * 1000.0 / 24576.0
CHAIN_US_PER_ROW_IDLE = 0.0303
CHAIN_US_PER_ROW_PRE_CORRECTION = 0.0875
CHAIN_US_PER_ROW_REMEASURED = 0.0987
CHAIN_FLOOR_MS = 0.248
CHAIN_LINEAR_MIN_ROWS = 24576
SECOND_ALPHA_PTS = [(8, 0.130), (16, 0.141), (32, 0.252), (64, 0.231), (128, 0.394)]
SECOND_BETA_FLAT = 111.9


def saturating_beta(beta_inf: float, x_half: float, lo: float = 1e3, hi: float = 1e9,
                    n: int = 48, floor: float = 1.0) -> list:
    """Table of beta(x) = beta_inf * x / (x + x_half): ``n`` log-spaced sizes on [lo, hi],
    continued downward with the same spacing to at or below ``floor`` bytes."""
    ratio = (hi / lo) ** (1.0 / (n - 1))
    sizes = [lo * ratio ** i for i in range(n)]
    x = lo / ratio
    while x > floor:
        sizes.insert(0, x)
        x /= ratio
    sizes.insert(0, x)
    if x_half <= 0:
        return [(s, beta_inf) for s in sizes]
    return [(s, beta_inf * s / (s + x_half)) for s in sizes]


def flat_supernode(x_half: float | None = None) -> ClusterSpec:
    flat = saturating_beta(BETA_FLAT, X_HALF_FLAT if x_half is None else x_half)
    return ClusterSpec(
        name="flat_supernode (calibrated from measurements)", R=8,
        fast=Level("node-internal", ALPHA_PTS, [(1e3, BETA_FAST), (1e9, BETA_FAST)]),
        slow=Level("cross-node", ALPHA_PTS, [(x, b * CROSS_NODE_RATIO) for x, b in flat]),
        flat=Level("full-fabric", ALPHA_PTS, flat),
        splits_sync_ms=SPLITS_SYNC_MS, chain_us_per_row=CHAIN_US_PER_ROW)


aug_flat = flat_supernode


def second_machine(x_half: float | None = None) -> ClusterSpec:
    beta = saturating_beta(SECOND_BETA_FLAT, X_HALF_FLAT if x_half is None else x_half)
    return ClusterSpec(
        name="second_machine (re-fitted from its own corpora)", R=8,
        fast=Level("node-internal", SECOND_ALPHA_PTS, beta),
        slow=Level("cross-node", SECOND_ALPHA_PTS, beta),
        flat=Level("full-fabric", SECOND_ALPHA_PTS, beta),
        splits_sync_ms=SPLITS_SYNC_MS, chain_us_per_row=CHAIN_US_PER_ROW)


def supernode_under_form(p: float, per_peer_us: float, beta_inf: float,
                         beta_fast: float | None = None, alpha_pts=None,
                         ratio: float = CROSS_NODE_RATIO) -> ClusterSpec:
    """Platform A under an alternative combination form: exponent ``p`` and an explicit per-peer
    message cost instead of the saturating bandwidth curve."""
    pts = alpha_pts or ALPHA_PTS
    flat = [(1.0, beta_inf), (1e12, beta_inf)]
    fast = [(1.0, beta_fast), (1e12, beta_fast)] if beta_fast else flat
    return ClusterSpec(
        name="supernode (p=%g)" % p, R=8,
        fast=Level("node-internal", pts, fast),
        slow=Level("cross-node", pts, [(x, b * ratio) for x, b in flat]),
        flat=Level("full-fabric", pts, flat),
        splits_sync_ms=SPLITS_SYNC_MS, chain_us_per_row=CHAIN_US_PER_ROW,
        combine_exponent=p, per_peer_us=per_peer_us)


def synthetic(ratio: float, name: str = "", R: int = 8, base_beta_gbps: float = 100.0,
              alpha_like_measured: bool = True, chain_us_per_row: float = CHAIN_US_PER_ROW,
              x_half: float = X_HALF_FLAT, **_compat) -> ClusterSpec:
    """Hypothetical machine whose slow level (and the flat fabric, set by the slow edge) is
    ``ratio`` times slower than the fast level."""
    alpha = ALPHA_PTS if alpha_like_measured else [(2, 0.05), (512, 0.05)]
    slow = saturating_beta(base_beta_gbps / ratio, x_half)
    return ClusterSpec(
        name=name or "synthetic(ratio=%.2f)" % ratio, R=R,
        fast=Level("fast", alpha, saturating_beta(base_beta_gbps, x_half)),
        slow=Level("slow", alpha, slow), flat=Level("flat", alpha, slow),
        splits_sync_ms=SPLITS_SYNC_MS, chain_us_per_row=chain_us_per_row)


# ---- platform B200 ----------------------------------------------------------------------------
# Defaults measured on 2 x B200 with the fused transport (dispatch+combine of 24576 rows of 8 KiB,
# half of them remote, took 0.36-0.38 ms).  ``b200_from_records`` replaces them with a fit.
B200_ALPHA_US = {"fast": 12.0, "slow": 12.0, "flat": 14.0}     # kernel launch + flag round trip
B200_BETA_GBPS = 650.0                                         # per direction, peer stores
B200_X_HALF = 16 * 1024
B200_CHAIN_US_PER_ROW = 0.0                                    # no arrival chain: rows are placed
B200_SPLITS_SYNC_MS = 0.0                                      # no host read-back


def b200_nvswitch(R: int = 2, alpha_us: dict | None = None, beta_gbps: float | None = None,
                  x_half: float | None = None, hop_overlap: float = 0.0,
                  chain_us_per_row: float = B200_CHAIN_US_PER_ROW) -> ClusterSpec:
    """8 x B200 behind one NVSwitch: the three levels share one port, so their bandwidths are
    equal and groups are logical; what differs is the per-exchange fixed cost."""
    a = dict(B200_ALPHA_US)
    a.update(alpha_us or {})
    beta = saturating_beta(beta_gbps or B200_BETA_GBPS, B200_X_HALF if x_half is None else x_half)

    def pts(us):
        return [(2, us / 1000.0), (16, us / 1000.0)]
    return ClusterSpec(
        name="b200_nvswitch", R=R,
        fast=Level("intra-group", pts(a["fast"]), beta),
        slow=Level("inter-group", pts(a["slow"]), beta),
        flat=Level("all ranks", pts(a["flat"]), beta),
        splits_sync_ms=B200_SPLITS_SYNC_MS, chain_us_per_row=chain_us_per_row,
        hop_overlap=hop_overlap)


def b200_from_records(records, R: int = 2) -> ClusterSpec:
    """Fit the B200 platform from sweep records ``{frame, world, bytes, ms}`` with frames
    ``fast`` / ``slow`` / ``flat`` (see ``sim.fit``): alpha pinned from the smallest message of
    every frame, (beta_inf, x_half) fitted on the rest."""
    from . import fit
    alpha_us = {}
    betas, halves = [], []
    for frame in ("fast", "slow", "flat"):
        recs = [r for r in records if r["frame"] == frame]
        if not recs:
            continue
        small = min(recs, key=lambda r: r["bytes"])
        alpha_us[frame] = small["ms"] * 1000.0
        res = fit.fit_beta_pinned(recs, lambda w, a=small["ms"]: a)
        betas.append(res["beta_inf"])
        halves.append(res["x_half"])
    beta = sum(betas) / len(betas) if betas else None
    x_half = sum(halves) / len(halves) if halves else None
    return b200_nvswitch(R=R, alpha_us=alpha_us, beta_gbps=beta, x_half=x_half)
