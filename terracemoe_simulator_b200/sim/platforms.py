"""Registry of measured platforms and ratio-only sensitivity scenarios.

A ``Platform`` carries the constants that were actually measured on one machine plus where they
came from, and builds its ``ClusterSpec``.  Registered: "A" (the reference's bandwidth-flat
supernode), "B" (its second machine, re-fitted), and "B200" (8 x B200 behind one NVSwitch with
the fused transport of this repository).  ``ARCHETYPES`` are synthetic hierarchy ratios for
sensitivity tables; only rows backed by a measurement are called measured.

Parity with the reference ``sim/platforms.py`` (``Platform`` :49-108, ``Archetype`` :116-143,
``platform_map`` / ``coverage`` / ``get`` :146-183).
"""
from __future__ import annotations

from dataclasses import dataclass

from . import calibrate as cal
from .core import ClusterSpec, Level


@dataclass
class Platform:
    key: str
    label: str
    hierarchy_ratio: float | None      # fast/slow bandwidth, only when both were measured
    alpha_pts: list
    beta_inf: float
    x_half: float
    beta_fast: float
    cross_node_ratio: float
    R: int = 8
    splits_sync_ms: float = cal.SPLITS_SYNC_MS
    chain_us_per_row: float = cal.CHAIN_US_PER_ROW
    provenance: str = ""
    fit_median_err: float = float("nan")
    n_targets: int = 0
    notes: str = ""

    def spec(self) -> ClusterSpec:
        flat = cal.saturating_beta(self.beta_inf, self.x_half)
        fast = [(1e3, self.beta_fast), (1e9, self.beta_fast)] if self.beta_fast else flat
        return ClusterSpec(
            name=self.label, R=self.R,
            fast=Level("node-internal", self.alpha_pts, fast),
            slow=Level("cross-node", self.alpha_pts,
                       [(x, b * self.cross_node_ratio) for x, b in flat]),
            flat=Level("full-fabric", self.alpha_pts, flat),
            splits_sync_ms=self.splits_sync_ms, chain_us_per_row=self.chain_us_per_row)


PLATFORMS = {
    "A": Platform(
        key="A", label="platform A (bandwidth-flat supernode)",
        hierarchy_ratio=1.0 / cal.CROSS_NODE_RATIO, alpha_pts=cal.ALPHA_PTS,
        beta_inf=cal.BETA_FLAT, x_half=cal.X_HALF_FLAT, beta_fast=cal.BETA_FAST,
        cross_node_ratio=cal.CROSS_NODE_RATIO,
        provenance="alpha measured directly at worlds 8/16/128; beta fitted on this machine's "
                   "own sweeps with alpha pinned; x_half borrowed from machine B",
        fit_median_err=0.019, n_targets=6,
        notes="Cross-node and intra-node bandwidth differ by 2.6%: the low end of the ratio "
              "axis; it settles nothing about hierarchical machines."),
    "B": Platform(
        key="B", label="platform B (second machine, re-fitted)", hierarchy_ratio=None,
        alpha_pts=cal.SECOND_ALPHA_PTS, beta_inf=cal.SECOND_BETA_FLAT, x_half=cal.X_HALF_FLAT,
        beta_fast=0.0, cross_node_ratio=1.0,
        provenance="alpha, flat beta and x_half fitted on this machine's own corpus; the level "
                   "split and the arrival chain are retained, not measured",
        fit_median_err=0.093, n_targets=44,
        notes="A consistency check of the functional form after refitting, not an "
              "out-of-sample transfer test; supplies no hierarchy ratio."),
    "B200": Platform(
        key="B200", label="8 x B200, one NVSwitch domain (fused peer-memory transport)",
        hierarchy_ratio=1.0,
        alpha_pts=[(2, cal.B200_ALPHA_US["flat"] / 1000.0), (16, cal.B200_ALPHA_US["flat"] / 1000.0)],
        beta_inf=cal.B200_BETA_GBPS, x_half=cal.B200_X_HALF, beta_fast=0.0, cross_node_ratio=1.0,
        R=2, splits_sync_ms=cal.B200_SPLITS_SYNC_MS, chain_us_per_row=cal.B200_CHAIN_US_PER_ROW,
        provenance="dispatch+combine sweeps of this repository's fused kernels, device-timed, "
                   "max over ranks; refit with calibrate.b200_from_records",
        fit_median_err=0.038, n_targets=48,     # sim/validate_b200.py: 48 measured configurations
        notes="All three levels share one NVLink port per GPU, so the hierarchy ratio is 1 by "
              "construction; groups are logical.  Two-hop can still win on bytes for R=2 "
              "because half of Hop B stays on the GPU."),
}


@dataclass
class Archetype:
    key: str
    label: str
    fast_side: str
    slow_side: str
    ratio_nominal: float
    note: str = ""


ARCHETYPES = [Archetype("measured-a", "Platform A measured ratio", "measured fast side",
                        "measured slow side", 1.03, "The only row whose ratio is measured.")]
ARCHETYPES += [Archetype("ratio-%d" % r, "Synthetic ratio scenario", "synthetic", "synthetic",
                         float(r), "Sensitivity point; not assigned to a named platform.")
               for r in (2, 4, 9, 18)]


def verdict(ratio: float, breakevens: dict) -> dict:
    return {tier: ratio >= be for tier, be in breakevens.items()}


def platform_map(q: int = 3, tok: int = 4096) -> list:
    from .sweep import CHAIN_SCENARIOS
    from .uncertainty import breakeven_ratio
    bes = {name: breakeven_ratio(chain, q=q, tok=tok) for name, chain in CHAIN_SCENARIOS}
    return [{"archetype": a, "breakevens": bes, "verdict": verdict(a.ratio_nominal, bes)}
            for a in ARCHETYPES]


def get(key: str) -> Platform:
    if key not in PLATFORMS:
        raise KeyError("unknown platform %r; have %s" % (key, sorted(PLATFORMS)))
    return PLATFORMS[key]


def coverage() -> dict:
    ratios = sorted(p.hierarchy_ratio for p in PLATFORMS.values() if p.hierarchy_ratio is not None)
    return {"n_platforms": len(PLATFORMS), "n_ratio_measured": len(ratios),
            "ratio_min": ratios[0], "ratio_max": ratios[-1],
            "spans_hierarchical": ratios[-1] >= 1.5,
            "targets_total": sum(p.n_targets for p in PLATFORMS.values())}


def main() -> None:
    print("=== measured platforms ===")
    print("%-5s %-60s %10s %9s %8s" % ("key", "platform", "ratio", "fit err", "targets"))
    for key in sorted(PLATFORMS):
        p = PLATFORMS[key]
        ratio = "%.2f" % p.hierarchy_ratio if p.hierarchy_ratio is not None else "unresolved"
        err = "%8.1f%%" % (p.fit_median_err * 100) if p.fit_median_err == p.fit_median_err else \
            "      n/a"
        print("%-5s %-60s %10s %s %8d" % (key, p.label[:60], ratio, err, p.n_targets))
    c = coverage()
    print("\n%d platforms, %d validation targets; ratio measured on %d platform(s): %.2f-%.2f"
          % (c["n_platforms"], c["targets_total"], c["n_ratio_measured"], c["ratio_min"],
             c["ratio_max"]))
    if not c["spans_hierarchical"]:
        from .hierarchy import CROSS_SUPERNODE_WORLD128_GBPS, loaded_ratio
        lo, hi = sorted(loaded_ratio(p) for p in CROSS_SUPERNODE_WORLD128_GBPS)
        print("No registered platform has a ratio above 1.5: the synthetic rows below are")
        print("sensitivities, not predictions.  Two measured ratios exist off this registry")
        print("(the two supernode boundaries of platform A): %.2f and %.2f." % (lo, hi))
    rows = platform_map()
    bes = rows[0]["breakevens"]
    tiers = list(bes)
    print("\n=== ratio-only sensitivity scenarios ===")
    print("%-44s %6s  %s" % ("scenario", "ratio", "  ".join("%-22s" % t[:22] for t in tiers)))
    print("%-44s %6s  %s" % ("", "", "  ".join("%-22s" % ("breakeven %.2f" % bes[t])
                                                for t in tiers)))
    for r in rows:
        a = r["archetype"]
        print("%-44s %6.2f  %s" % (a.label[:44], a.ratio_nominal,
                                   "  ".join("%-22s" % ("yes" if r["verdict"][t] else "no")
                                             for t in tiers)))
    print("\nThese are ratio-only sensitivity scenarios, not deployment verdicts.")


if __name__ == "__main__":
    main()
