"""Machine checklist: does a machine / geometry qualify for the two-hop dispatch, and why.

``check`` returns six named conditions (quota, effective breakeven against the hierarchy ratio,
EP spanning more than one fast domain, bandwidth-bound messages, fixed cost of two small
exchanges against one large one, arrival-chain tier); ``profile_from_spec`` adds the full
model's ratio so the checklist can never silently contradict it.  Also: measured launch
constants of platform A and two sensitivity scans (extra launch latency, per-world bandwidth).

Parity with the reference ``sim/profile.py`` (``Condition`` :56-61, ``byte_breakeven`` :71-75,
``check`` :78-155, launch constants :162-222, ``launch_sensitivity`` :226-272,
``bandwidth_world_sensitivity`` :275-347, ``verdict`` / ``profile_from_spec`` :350-370).
"""
from __future__ import annotations

from dataclasses import dataclass

from .core import ClusterSpec, Level, MoEGeometry, one_hop_call, two_hop_call

FUSED_TIER_US = 0.02
FUSED_TARGET_US = 0.012


@dataclass
class Condition:
    name: str
    passed: bool
    detail: str
    margin: float = float("nan")      # > 0 passes; magnitude = headroom


def byte_breakeven(R: int, q: int) -> float:
    """Hierarchy ratio at which the two-hop byte ledger alone breaks even."""
    if q <= 1:
        return float("inf")
    return (1.0 - 1.0 / R) * q / (q - 1)


def check(ratio: float, R: int, k: int, M: int, ep: int, tokens_per_rank: int, hidden: int,
          chain_us_per_row: float, alpha_of_world=None, x_half_bytes: float = 54 * 1024,
          bytes_per_elem: int = 2) -> list:
    from .uncertainty import breakeven_ratio
    q = k // M if M else 0
    n_groups = max(ep // R, 1)
    inf = float("inf")
    out = [Condition("q = k/M >= 2", q >= 2,
                     "q=%d (k=%d, M=%d); the slow-side saving is (q-1)/q = %.0f%%"
                     % (q, k, M, 100 * (q - 1) / q if q else 0), margin=q - 2)]
    be_bytes = byte_breakeven(R, q) if q >= 2 else inf
    be_eff = breakeven_ratio(chain_us_per_row, q=q, tok=tokens_per_rank) if q >= 2 else inf
    out.append(Condition(
        "hierarchy ratio beats the effective breakeven", ratio >= be_eff,
        "ratio %.2f vs effective breakeven %.2f (bytes alone would need %.2f; the gap is what "
        "the arrival chain costs)" % (ratio, be_eff, be_bytes), margin=ratio - be_eff))
    out.append(Condition(
        "EP spans more than one fast domain", n_groups >= 2,
        "EP=%d over domains of %d cards = %d group(s)%s"
        % (ep, R, n_groups, "" if n_groups >= 2 else " -- keep EP inside the domain instead"),
        margin=n_groups - 2))
    per_peer = tokens_per_rank * k * hidden * bytes_per_elem / max(ep, 1)
    out.append(Condition(
        "messages are bandwidth-bound", per_peer >= 4 * x_half_bytes,
        "one-hop per-peer %.0f KiB vs half-performance size %.0f KiB (want >=4x)"
        % (per_peer / 1024, x_half_bytes / 1024), margin=per_peer / x_half_bytes - 4))
    name = "fixed cost: two small collectives beat one big one"
    if alpha_of_world is None:
        out.append(Condition(name, False, "UNKNOWN -- supply the machine's measured "
                                          "alpha(world); it cannot be assumed"))
    else:
        two, one = alpha_of_world(n_groups) + alpha_of_world(R), alpha_of_world(ep)
        out.append(Condition(name, two < one, "alpha(%d)+alpha(%d) = %.3f ms vs alpha(%d) = "
                             "%.3f ms" % (n_groups, R, two, ep, one), margin=one - two))
    fused = chain_us_per_row <= FUSED_TIER_US
    be_fused = breakeven_ratio(FUSED_TARGET_US, q=q, tok=tokens_per_rank) if q >= 2 else inf
    note = ("fused tier; the threshold is as low as this model goes" if fused else
            "an op chain: it raises the breakeven from %.2f (fused) to %.2f, so fusing it is "
            "worth more than most topology changes" % (be_fused, be_eff))
    out.append(Condition("arrival chain cost (advisory, already priced above)", True,
                         "%.4f us/row -- %s" % (chain_us_per_row, note),
                         margin=FUSED_TIER_US - chain_us_per_row))
    return out


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


def _breakeven(speedup, steps: int = 40, lo: float = 1.0, hi: float = 32.0) -> float:
    if speedup(lo) >= 1.0:
        return lo
    if speedup(hi) < 1.0:
        return hi
    for _ in range(steps):
        mid = (lo + hi) / 2.0
        if speedup(mid) >= 1.0:
            hi = mid
        else:
            lo = mid
    return hi


def launch_sensitivity(geom, chain_us_per_row: float,
                       deltas_ms=(0.0, 0.04, 0.08, 0.111, 0.130, 0.16, 0.25)) -> list:
    """How the breakeven moves when every two-hop call pays ``d`` ms of extra launch latency."""
    from .calibrate import synthetic
    out = []
    for d in deltas_ms:
        def ratio(r, d=d):
            c = synthetic(r, chain_us_per_row=chain_us_per_row)
            return one_hop_call(c, geom) / (two_hop_call(c, geom) + d)
        out.append({"extra_launch_ms": d, "breakeven": _breakeven(ratio),
                    "ratio_at_3.2": ratio(3.2), "ratio_at_8": ratio(8.0)})
    return out


def bandwidth_world_sensitivity(geom=None, chain_us_per_row: float | None = None) -> list:
    """Breakeven with one bandwidth for all worlds against the measured per-world marginal
    bandwidths (fast: world 8, slow: world 16, flat: world 128)."""
    from .calibrate import BETA_FLAT, MARGINAL_BW_BY_WORLD, synthetic
    from .sweep import CHAIN_SCENARIOS
    g = geom or MoEGeometry(name="ref", n_groups=16, R=8, k=6, M=2, H=2048, seq=4096, mbs=1,
                            gbs=16 * 8 * 4096)
    tiers = list(CHAIN_SCENARIOS) if chain_us_per_row is None else [("supplied", chain_us_per_row)]

    def spec(ratio, chain, per_world):
        c = synthetic(ratio, chain_us_per_row=chain)
        if not per_world:
            return c

        def scaled(level, world):
            return [(x, b * MARGINAL_BW_BY_WORLD[world] / BETA_FLAT) for x, b in level.beta_pts]
        return ClusterSpec(name=c.name + " + per-world bandwidth", R=c.R,
                           fast=Level("fast", c.fast.alpha_pts, scaled(c.fast, 8)),
                           slow=Level("slow", c.slow.alpha_pts, scaled(c.slow, 16)),
                           flat=Level("flat", c.flat.alpha_pts, scaled(c.flat, 128)),
                           splits_sync_ms=c.splits_sync_ms, chain_us_per_row=c.chain_us_per_row)

    def be(chain, per_world):
        def s(r):
            c = spec(r, chain, per_world)
            return one_hop_call(c, g) / two_hop_call(c, g)
        return _breakeven(s, steps=50)
    return [(name, be(chain, False), be(chain, True)) for name, chain in tiers]


def verdict(conditions) -> dict:
    failed = [c for c in conditions if not c.passed]
    return {"qualifies": not failed, "n_failed": len(failed),
            "first_failure": failed[0].name if failed else None}


def profile_from_spec(cluster, geom: MoEGeometry, ratio: float | None = None) -> dict:
    r = ratio if ratio is not None else cluster.ratio()
    conds = check(ratio=r, R=geom.R, k=geom.k, M=geom.M, ep=geom.ep,
                  tokens_per_rank=geom.tokens_per_rank, hidden=geom.H,
                  chain_us_per_row=cluster.chain_us_per_row, alpha_of_world=cluster.flat.alpha_ms)
    return {"conditions": conds, "verdict": verdict(conds),
            "model_ratio": one_hop_call(cluster, geom) / two_hop_call(cluster, geom)}


def main() -> None:
    from .calibrate import b200_nvswitch, flat_supernode, synthetic
    from .sweep import CHAIN_SCENARIOS
    g = MoEGeometry(name="op", n_groups=16, R=8, k=6, M=2, seq=4096, mbs=1, gbs=16 * 8 * 4096)
    g_b200 = MoEGeometry(name="b200", n_groups=4, R=2, k=6, M=2, H=4096, seq=4096, mbs=1,
                         gbs=8 * 4096)
    cases = [("platform A, as measured", flat_supernode(), None, g),
             ("NVLink+IB class, PyTorch chain",
              synthetic(9.0, chain_us_per_row=CHAIN_SCENARIOS[0][1]), 9.0, g),
             ("NVLink+IB class, fused chain",
              synthetic(9.0, chain_us_per_row=CHAIN_SCENARIOS[1][1]), 9.0, g),
             ("8 x B200, one NVSwitch domain, fused transport", b200_nvswitch(R=2), None, g_b200)]
    for label, spec, ratio, geom in cases:
        r = profile_from_spec(spec, geom, ratio)
        print("=== %s ===" % label)
        for c in r["conditions"]:
            print("  [%s] %-48s %s" % ("PASS" if c.passed else "FAIL", c.name, c.detail))
        v = r["verdict"]
        print("  -> %s;  full model says one-hop/two-hop = %.2f\n"
              % ("qualifies" if v["qualifies"] else
                 "does not qualify (first failure: %s)" % v["first_failure"], r["model_ratio"]))
    print("The checklist is necessary conditions; the model ratio is what they add up to.")
    print("When they disagree, read the condition that fails: it names the reason.")


if __name__ == "__main__":
    main()
