"""Machine checklist: does a machine / geometry qualify for the two-hop dispatch, and why.

A ``Subject`` gathers what the rules look at (hierarchy ratio, group size, routing shape, tokens
per rank, hidden width, arrival-chain cost, the machine's fixed cost per exchange as a function
of the number of peers).  Six rules, applied in a fixed order, each return one ``Condition``:
the quota is at least two; the ratio beats the effective breakeven (bytes plus what the arrival
chain costs); expert parallelism spans more than one fast domain; messages are bandwidth bound;
two small exchanges cost less fixed time than one large one; and, as advice, which arrival-chain
tier the machine sits on.  ``profile_from_spec`` puts the full model's ratio beside the
checklist so that the two can never silently disagree.  Also here: two sensitivity scans of the
breakeven ratio (extra launch latency per call; one bandwidth for all worlds against measured
per-world bandwidths), both through one bisection helper.

Public surface of the reference's ``sim/profile.py`` (``Condition`` :56-61, ``byte_breakeven``
:71-75, ``check`` :78-155, launch constants :162-222, ``launch_sensitivity`` :226-272,
``bandwidth_world_sensitivity`` :275-347, ``verdict`` / ``profile_from_spec`` :350-370).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

from .core import ClusterSpec, Level, MoEGeometry, one_hop_call, two_hop_call
from .records import (HOST_EXPOSURE_MS, HOST_SUBMIT_MS, LAUNCH_DEVICE_INITIATED_MS,  # noqa: F401
                      LAUNCH_HOST_P2P_MS, LAUNCH_UPPER_BOUND_MS, PER_CALL_DEEP_QUEUE_MS,
                      PER_CALL_DEEP_QUEUE_RANGE_MS, PER_CALL_HOST_EXPOSED_MS, PER_CALL_SPREAD)

FUSED_TIER_US = 0.02
FUSED_TARGET_US = 0.012
INF = float("inf")


@dataclass
class Condition:
    name: str
    passed: bool
    detail: str
    margin: float = float("nan")      # > 0 passes; magnitude = headroom


def byte_breakeven(R: int, q: int) -> float:
    """Hierarchy ratio at which the two-hop byte ledger alone breaks even."""
    return INF if q <= 1 else q * (R - 1) / (R * (q - 1.0))


@dataclass(frozen=True)
class Subject:
    ratio: float
    R: int
    k: int
    M: int
    ep: int
    tokens_per_rank: int
    hidden: int
    chain_us_per_row: float
    alpha_of_world: Optional[Callable] = None
    x_half_bytes: float = 54 * 1024
    bytes_per_elem: int = 2

    @property
    def q(self) -> int:
        return self.k // self.M if self.M else 0

    @property
    def n_groups(self) -> int:
        return self.ep // self.R or 1

    @property
    def per_peer_bytes(self) -> float:
        return self.tokens_per_rank * self.k * self.hidden * self.bytes_per_elem / (self.ep or 1)

    def effective_breakeven(self, chain_us: float | None = None) -> float:
        if self.q < 2:
            return INF
        from .uncertainty import breakeven_ratio
        chain = self.chain_us_per_row if chain_us is None else chain_us
        return breakeven_ratio(chain, q=self.q, tok=self.tokens_per_rank)


def _rule_quota(s: Subject) -> Condition:
    saved = 100 * (s.q - 1) / s.q if s.q else 0
    return Condition("q = k/M >= 2", s.q >= 2,
                     "q=%d (k=%d, M=%d); the slow-side saving is (q-1)/q = %.0f%%"
                     % (s.q, s.k, s.M, saved), margin=s.q - 2)


def _rule_ratio(s: Subject) -> Condition:
    need = s.effective_breakeven()
    bytes_only = byte_breakeven(s.R, s.q) if s.q >= 2 else INF
    return Condition("hierarchy ratio beats the effective breakeven", s.ratio >= need,
                     "ratio %.2f vs effective breakeven %.2f (bytes alone would need %.2f; the "
                     "gap is what the arrival chain costs)" % (s.ratio, need, bytes_only),
                     margin=s.ratio - need)


def _rule_domains(s: Subject) -> Condition:
    spans = s.n_groups >= 2
    hint = "" if spans else " -- keep EP inside the domain instead"
    return Condition("EP spans more than one fast domain", spans,
                     "EP=%d over domains of %d cards = %d group(s)%s"
                     % (s.ep, s.R, s.n_groups, hint), margin=s.n_groups - 2)


def _rule_message_size(s: Subject) -> Condition:
    multiple = s.per_peer_bytes / s.x_half_bytes
    return Condition("messages are bandwidth-bound", multiple >= 4,
                     "one-hop per-peer %.0f KiB vs half-performance size %.0f KiB (want >=4x)"
                     % (s.per_peer_bytes / 1024, s.x_half_bytes / 1024), margin=multiple - 4)


def _rule_fixed_cost(s: Subject) -> Condition:
    name = "fixed cost: two small collectives beat one big one"
    alpha = s.alpha_of_world
    if alpha is None:
        return Condition(name, False, "UNKNOWN -- supply the machine's measured alpha(world); it "
                                      "cannot be assumed")
    split, whole = alpha(s.n_groups) + alpha(s.R), alpha(s.ep)
    return Condition(name, split < whole, "alpha(%d)+alpha(%d) = %.3f ms vs alpha(%d) = %.3f ms"
                     % (s.n_groups, s.R, split, s.ep, whole), margin=whole - split)


def _rule_chain_tier(s: Subject) -> Condition:
    if s.chain_us_per_row <= FUSED_TIER_US:
        note = "fused tier; the threshold is as low as this model goes"
    else:
        note = ("an op chain: it raises the breakeven from %.2f (fused) to %.2f, so fusing it is "
                "worth more than most topology changes"
                % (s.effective_breakeven(FUSED_TARGET_US), s.effective_breakeven()))
    return Condition("arrival chain cost (advisory, already priced above)", True,
                     "%.4f us/row -- %s" % (s.chain_us_per_row, note),
                     margin=FUSED_TIER_US - s.chain_us_per_row)


RULES = (_rule_quota, _rule_ratio, _rule_domains, _rule_message_size, _rule_fixed_cost,
         _rule_chain_tier)


def check(ratio: float, R: int, k: int, M: int, ep: int, tokens_per_rank: int, hidden: int,
          chain_us_per_row: float, alpha_of_world=None, x_half_bytes: float = 54 * 1024,
          bytes_per_elem: int = 2) -> list:
    subject = Subject(ratio, R, k, M, ep, tokens_per_rank, hidden, chain_us_per_row,
                      alpha_of_world, x_half_bytes, bytes_per_elem)
    return [rule(subject) for rule in RULES]


def _breakeven(speedup, steps: int = 40, lo: float = 1.0, hi: float = 32.0) -> float:
    """Smallest hierarchy ratio in [lo, hi] at which ``speedup(ratio) >= 1`` (bisection on a
    function that grows with the ratio); ``lo`` or ``hi`` when the crossing lies outside."""
    if speedup(lo) >= 1.0:
        return lo
    if speedup(hi) < 1.0:
        return hi
    for _ in range(steps):
        mid = 0.5 * (lo + hi)
        lo, hi = (lo, mid) if speedup(mid) >= 1.0 else (mid, hi)
    return hi


def launch_sensitivity(geom, chain_us_per_row: float,
                       deltas_ms=(0.0, 0.04, 0.08, 0.111, 0.130, 0.16, 0.25)) -> list:
    """How the breakeven moves when every two-hop call pays ``d`` ms of extra launch latency."""
    from .calibrate import synthetic

    def speedup_with(extra_ms: float):
        def speedup(ratio: float) -> float:
            cluster = synthetic(ratio, chain_us_per_row=chain_us_per_row)
            return one_hop_call(cluster, geom) / (two_hop_call(cluster, geom) + extra_ms)
        return speedup

    rows = []
    for extra in deltas_ms:
        f = speedup_with(extra)
        rows.append({"extra_launch_ms": extra, "breakeven": _breakeven(f), "ratio_at_3.2": f(3.2),
                     "ratio_at_8": f(8.0)})
    return rows


_LEVEL_WORLD = (("fast", 8), ("slow", 16), ("flat", 128))     # world each level was measured at


def _with_per_world_bandwidth(cluster: ClusterSpec) -> ClusterSpec:
    """``cluster`` with every level's bandwidth curve rescaled to the marginal bandwidth measured
    at that level's world size."""
    from .calibrate import BETA_FLAT, MARGINAL_BW_BY_WORLD
    levels = {}
    for name, world in _LEVEL_WORLD:
        level = getattr(cluster, name)
        gain = MARGINAL_BW_BY_WORLD[world] / BETA_FLAT
        levels[name] = Level(name, level.alpha_pts, [(x, b * gain) for x, b in level.beta_pts])
    return ClusterSpec(name=cluster.name + " + per-world bandwidth", R=cluster.R,
                       splits_sync_ms=cluster.splits_sync_ms,
                       chain_us_per_row=cluster.chain_us_per_row, **levels)


def bandwidth_world_sensitivity(geom=None, chain_us_per_row: float | None = None) -> list:
    """Breakeven with one bandwidth for all worlds against the measured per-world marginal
    bandwidths (fast: world 8, slow: world 16, flat: world 128)."""
    from .calibrate import synthetic
    from .sweep import CHAIN_SCENARIOS
    g = geom or MoEGeometry(name="ref", n_groups=16, R=8, k=6, M=2, H=2048, seq=4096, mbs=1,
                            gbs=16 * 8 * 4096)
    tiers = [("supplied", chain_us_per_row)] if chain_us_per_row is not None \
        else list(CHAIN_SCENARIOS)

    def crossing(chain: float, per_world: bool) -> float:
        def speedup(ratio: float) -> float:
            cluster = synthetic(ratio, chain_us_per_row=chain)
            if per_world:
                cluster = _with_per_world_bandwidth(cluster)
            return one_hop_call(cluster, g) / two_hop_call(cluster, g)
        return _breakeven(speedup, steps=50)

    return [(name, crossing(chain, False), crossing(chain, True)) for name, chain in tiers]


def verdict(conditions) -> dict:
    failing = [c.name for c in conditions if not c.passed]
    return {"qualifies": not failing, "n_failed": len(failing),
            "first_failure": failing[0] if failing else None}


def profile_from_spec(cluster, geom: MoEGeometry, ratio: float | None = None) -> dict:
    conditions = check(ratio=cluster.ratio() if ratio is None else ratio, R=geom.R, k=geom.k,
                       M=geom.M, ep=geom.ep, tokens_per_rank=geom.tokens_per_rank, hidden=geom.H,
                       chain_us_per_row=cluster.chain_us_per_row,
                       alpha_of_world=cluster.flat.alpha_ms)
    return {"conditions": conditions, "verdict": verdict(conditions),
            "model_ratio": one_hop_call(cluster, geom) / two_hop_call(cluster, geom)}


def _cases():
    from .calibrate import b200_nvswitch, flat_supernode, synthetic
    from .sweep import CHAIN_SCENARIOS
    wide = MoEGeometry(name="op", n_groups=16, R=8, k=6, M=2, seq=4096, mbs=1, gbs=16 * 8 * 4096)
    box = MoEGeometry(name="b200", n_groups=4, R=2, k=6, M=2, H=4096, seq=4096, mbs=1,
                      gbs=8 * 4096)
    yield "platform A, as measured", flat_supernode(), None, wide
    for label, (_tier, chain) in zip(("PyTorch", "fused"), CHAIN_SCENARIOS):
        yield ("NVLink+IB class, %s chain" % label, synthetic(9.0, chain_us_per_row=chain), 9.0,
               wide)
    yield "8 x B200, one NVSwitch domain, fused transport", b200_nvswitch(R=2), None, box


def main() -> None:
    for label, spec, ratio, geom in _cases():
        result = profile_from_spec(spec, geom, ratio)
        print("=== %s ===" % label)
        for c in result["conditions"]:
            print("  [%s] %-48s %s" % ("PASS" if c.passed else "FAIL", c.name, c.detail))
        v = result["verdict"]
        outcome = "qualifies" if v["qualifies"] else \
            "does not qualify (first failure: %s)" % v["first_failure"]
        print("  -> %s;  full model says one-hop/two-hop = %.2f\n" % (outcome, result["model_ratio"]))
    print("The checklist is necessary conditions; the model ratio is what they add up to.")
    print("When they disagree, read the condition that fails: it names the reason.")


if __name__ == "__main__":
    main()
