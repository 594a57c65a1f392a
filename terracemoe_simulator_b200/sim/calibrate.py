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
# Constants fitted (``b200_from_sweep``) on the 48-point dispatch+combine sweep measured on
# 8 x B200 with the fused transport (``sim/data/b200_sweep_8gpu.json``; rows of 8 KiB, 256-16384
# tokens per GPU, R in {1, 2, 4}, q in {1..4}; device-timed, max over ranks, median of three
# bursts).  One exchange = half of a measured dispatch+combine.
B200_ALPHA_ONE_HOP_MS = 0.0355        # fixed cost of a one-hop exchange (plan + push/pull + flags)
B200_ALPHA_SLOW_MS = 0.0309           # Hop A of a two-hop exchange
B200_ALPHA_FAST_MS = 0.0300           # Hop B when it crosses GPUs (groups of two or more)
B200_ALPHA_FAST_LOCAL_MS = 0.0215     # Hop B inside one GPU (groups of one): no peer flags to wait for
B200_ALPHA_TWO_HOP_MS = B200_ALPHA_SLOW_MS + B200_ALPHA_FAST_MS     # both hops, groups of >= 2
B200_BETA_GBPS = 647.0                # NVLink payload bandwidth per direction, peer stores/loads
B200_SELF_COPY_GBPS = 2480.0          # rows that stay on the GPU: read + write through HBM
B200_SELF_OVERLAP_P = 1.5             # wire and local traffic overlap partly inside one kernel
B200_X_HALF = 0.0
B200_CHAIN_US_PER_ROW = 0.0           # no arrival chain: rows are stored at their final place
B200_SPLITS_SYNC_MS = 0.0             # no host read-back
B200_ALPHA_US = {"fast": B200_ALPHA_FAST_MS * 1000.0, "slow": B200_ALPHA_SLOW_MS * 1000.0,
                 "flat": B200_ALPHA_ONE_HOP_MS * 1000.0}


def b200_nvswitch(R: int = 2, alpha_one_ms: float = B200_ALPHA_ONE_HOP_MS,
                  alpha_slow_ms: float = B200_ALPHA_SLOW_MS,
                  alpha_fast_ms: float = B200_ALPHA_FAST_MS,
                  alpha_fast_local_ms: float = B200_ALPHA_FAST_LOCAL_MS,
                  beta_gbps: float = B200_BETA_GBPS,
                  self_copy_gbps: float = B200_SELF_COPY_GBPS,
                  self_overlap_p: float = B200_SELF_OVERLAP_P, hop_overlap: float = 0.0,
                  chain_us_per_row: float = B200_CHAIN_US_PER_ROW) -> ClusterSpec:
    """8 x B200 behind one NVSwitch: the three levels share one port per GPU, so their
    bandwidths are equal and groups are logical; what differs is the per-exchange fixed cost.
    Hop B has two of them: with groups of one GPU it never leaves the GPU (a local expansion
    that waits for no peer), with larger groups it is a real exchange.  Rows whose destination
    is the sending GPU are priced as a local copy."""
    beta = [(1.0, beta_gbps), (1e12, beta_gbps)]

    def flat(ms):
        return [(1, ms), (16, ms)]
    return ClusterSpec(
        name="b200_nvswitch", R=R,
        fast=Level("intra-group", [(1, alpha_fast_local_ms), (2, alpha_fast_ms), (16, alpha_fast_ms)],
                   beta),
        slow=Level("inter-group", flat(alpha_slow_ms), beta),
        flat=Level("all ranks", flat(alpha_one_ms), beta),
        splits_sync_ms=B200_SPLITS_SYNC_MS, chain_us_per_row=chain_us_per_row,
        hop_overlap=hop_overlap, self_copy_gbps=self_copy_gbps, self_overlap_p=self_overlap_p)


def load_b200_sweep(path: str | None = None) -> list:
    """Rows of the committed 8-GPU sweep (or of another sweep JSON written by ``bench/sweep.py``)."""
    import json
    import os
    if path is None:
        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data",
                            "b200_sweep_8gpu.json")
    with open(path, encoding="utf-8") as fh:
        return json.load(fh)["rows"]


def _sweep_geometry(row: dict):
    from .core import MoEGeometry
    T = row["tokens"]
    return MoEGeometry(name="sweep", n_groups=row["n_groups"], R=row["R"], k=row["k"], M=row["M"],
                       H=row["hidden"], seq=T, mbs=1, gbs=row["n_groups"] * row["R"] * T)


def b200_from_sweep(rows, overlap_p: float = B200_SELF_OVERLAP_P) -> ClusterSpec:
    """Fit of the six constants of ``b200_nvswitch`` (fixed costs of one-hop, Hop A, remote and
    local Hop B; link bandwidth; local-copy bandwidth) to sweep rows with measured
    ``one_hop_ms`` / ``two_hop_ms`` (dispatch + combine = two exchanges each).  Relative
    residuals with a soft-L1 loss: a 50 us call that one burst caught at twice its time must not
    move the constants.  Needs scipy."""
    import numpy as np
    from scipy.optimize import least_squares
    from .core import one_hop_call, two_hop_call
    geoms = [_sweep_geometry(r) for r in rows]
    target = np.array([v for r in rows for v in (r["one_hop_ms"] / 2, r["two_hop_ms"] / 2)])
    names = ("alpha_one_ms", "alpha_slow_ms", "alpha_fast_ms", "alpha_fast_local_ms", "beta_gbps",
             "self_copy_gbps")
    has = {bool(g.R == 1) for g in geoms}

    def spec(p):
        kw = dict(zip(names, (float(v) for v in p)))
        if has == {True}:                     # only groups of one GPU: the remote cost is unseen
            kw["alpha_fast_ms"] = kw["alpha_fast_local_ms"]
        elif has == {False}:
            kw["alpha_fast_local_ms"] = kw["alpha_fast_ms"]
        return b200_nvswitch(self_overlap_p=overlap_p, **kw)

    def residual(p):
        c = spec(p)
        model = np.array([v for g in geoms for v in (one_hop_call(c, g), two_hop_call(c, g))])
        return (model - target) / target

    sol = least_squares(residual, [0.04, 0.03, 0.03, 0.02, 650.0, 2500.0], loss="soft_l1",
                        f_scale=0.1, bounds=([0.0] * 4 + [50.0, 100.0], [1.0] * 4 + [2000.0, 20000.0]))
    return spec(sol.x)


def b200_from_records(records, R: int = 2) -> ClusterSpec:
    """Per-level fit from ``{frame, world, bytes, ms}`` records as written by ``bench/sweep.py``
    (frames ``flat``, ``slow``, ``fast``; ``slow`` / ``fast`` records carry the group size ``R``
    they were measured with).  Every frame gets its own fixed cost -- the time of its smallest
    message, per peer-set size -- and its own bandwidth curve from ``fit.fit_beta_pinned``.  A
    frame without records inherits the flat level's fit (or the shipped constants)."""
    from . import fit

    def pick(frame):
        out = []
        for r in records:
            r = r if isinstance(r, dict) else dict(zip(("frame", "world", "bytes", "ms"), r))
            if r["frame"] == frame and (frame == "flat" or r.get("R", R) == R):
                out.append(r)
        return out

    def level(name, recs, fallback):
        if len(recs) < 3:
            return fallback
        by_world: dict = {}
        for r in recs:
            w = int(r["world"])
            if w not in by_world or r["bytes"] < by_world[w][0]:
                by_world[w] = (r["bytes"], r["ms"])
        alpha_pts = sorted((w, ms) for w, (_b, ms) in by_world.items())
        alpha = Level(name, alpha_pts if len(alpha_pts) > 1 else
                      [(1, alpha_pts[0][1]), (16, alpha_pts[0][1])], [(1.0, 1.0), (1e12, 1.0)])
        res = fit.fit_beta_pinned(recs, alpha.alpha_ms)
        return Level(name, alpha.alpha_pts, saturating_beta(res["beta_inf"], res["x_half"]))

    base = b200_nvswitch(R=R)
    flat = level("all ranks", pick("flat"), base.flat)
    inherit_beta = flat.beta_pts
    fast = level("intra-group", pick("fast"), Level("intra-group", base.fast.alpha_pts, inherit_beta))
    slow = level("inter-group", pick("slow"), Level("inter-group", base.slow.alpha_pts, inherit_beta))
    return ClusterSpec(name="b200_nvswitch (per-level fit)", R=R, fast=fast, slow=slow, flat=flat,
                       splits_sync_ms=B200_SPLITS_SYNC_MS, chain_us_per_row=B200_CHAIN_US_PER_ROW,
                       self_copy_gbps=B200_SELF_COPY_GBPS, self_overlap_p=B200_SELF_OVERLAP_P)


def load_b200_records(path: str | None = None) -> list:
    """``records`` of a sweep JSON (default: the committed 8-GPU sweep)."""
    import json
    import os
    if path is None:
        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data",
                            "b200_sweep_8gpu.json")
    with open(path, encoding="utf-8") as fh:
        return json.load(fh).get("records", [])
