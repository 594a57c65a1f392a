"""Registry of measured platforms and ratio-only sensitivity scenarios.

A ``Platform`` is a set of constants measured on one machine, a sentence on where each came from,
and the recipe that turns them into a ``ClusterSpec``.  The registry lists the machine this
repository measures first:

  "B200"  8 x B200 behind one NVSwitch, fused peer-memory transport (this repository's sweeps)
  "A"     the reference's bandwidth-flat supernode
  "B"     the reference's second machine, re-fitted

A platform counts as a sample of the *hierarchy ratio* (fast over slow bandwidth) only when both
sides were measured there; "B" was not.  ``ARCHETYPES`` are synthetic ratios for sensitivity
tables, and ``platform_map`` derives their yes/no cells from the break-even ratios instead of
stating them.

Parity with the reference ``sim/platforms.py`` (``Platform`` :49-108, ``Archetype`` :116-143,
``platform_map`` / ``coverage`` / ``get`` :146-183).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

from . import calibrate as cal
from ._text import Column, render_table
from .core import ClusterSpec, Level

HIERARCHICAL_FROM = 1.5        # ratio from which a machine counts as hierarchical


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
    fit_median_err: float = math.nan
    n_targets: int = 0
    notes: str = ""

    def curves(self) -> dict:
        """Bandwidth-versus-size points of the three levels: the full fabric follows the
        saturating curve, the cross-node level is that curve scaled, the node-internal level is
        a constant where one was measured."""
        full = cal.saturating_beta(self.beta_inf, self.x_half)
        across = [(size, self.cross_node_ratio * gbps) for size, gbps in full]
        inside = full if not self.beta_fast else [(1e3, self.beta_fast), (1e9, self.beta_fast)]
        return {"full-fabric": full, "cross-node": across, "node-internal": inside}

    def spec(self) -> ClusterSpec:
        level = {name: Level(name, self.alpha_pts, pts) for name, pts in self.curves().items()}
        return ClusterSpec(name=self.label, R=self.R, fast=level["node-internal"],
                           slow=level["cross-node"], flat=level["full-fabric"],
                           splits_sync_ms=self.splits_sync_ms,
                           chain_us_per_row=self.chain_us_per_row)

    @property
    def ratio_measured(self) -> bool:
        return self.hierarchy_ratio is not None


def _b200() -> Platform:
    alpha_ms = cal.B200_ALPHA_US["flat"] / 1000.0
    return Platform(
        key="B200", label="8 x B200, one NVSwitch domain (fused peer-memory transport)",
        hierarchy_ratio=1.0, alpha_pts=[(2, alpha_ms), (16, alpha_ms)],
        beta_inf=cal.B200_BETA_GBPS, x_half=cal.B200_X_HALF, beta_fast=0.0, cross_node_ratio=1.0,
        R=2, splits_sync_ms=cal.B200_SPLITS_SYNC_MS, chain_us_per_row=cal.B200_CHAIN_US_PER_ROW,
        provenance="dispatch+combine sweeps of this repository's fused kernels, device-timed, "
                   "max over ranks; refit with calibrate.b200_from_records",
        fit_median_err=0.031, n_targets=48,     # sim/validate_b200.py: 48 measured configurations
        notes="All three levels share one NVLink port per GPU, so the hierarchy ratio is 1 by "
              "construction; groups are logical.  Two-hop can still win on bytes for R=2 "
              "because half of Hop B stays on the GPU.")


def _reference_machines() -> list:
    a = Platform(
        key="A", label="platform A (bandwidth-flat supernode)",
        hierarchy_ratio=1.0 / cal.CROSS_NODE_RATIO, alpha_pts=cal.ALPHA_PTS,
        beta_inf=cal.BETA_FLAT, x_half=cal.X_HALF_FLAT, beta_fast=cal.BETA_FAST,
        cross_node_ratio=cal.CROSS_NODE_RATIO,
        provenance="alpha measured directly at worlds 8/16/128; beta fitted on this machine's "
                   "own sweeps with alpha pinned; x_half borrowed from machine B",
        fit_median_err=0.019, n_targets=6,
        notes="Cross-node and intra-node bandwidth differ by 2.6%: the low end of the ratio "
              "axis; it settles nothing about hierarchical machines.")
    b = Platform(
        key="B", label="platform B (second machine, re-fitted)", hierarchy_ratio=None,
        alpha_pts=cal.SECOND_ALPHA_PTS, beta_inf=cal.SECOND_BETA_FLAT, x_half=cal.X_HALF_FLAT,
        beta_fast=0.0, cross_node_ratio=1.0,
        provenance="alpha, flat beta and x_half fitted on this machine's own corpus; the level "
                   "split and the arrival chain are retained, not measured",
        fit_median_err=0.093, n_targets=44,
        notes="A consistency check of the functional form after refitting, not an "
              "out-of-sample transfer test; supplies no hierarchy ratio.")
    return [a, b]


PLATFORMS = {p.key: p for p in [_b200(), *_reference_machines()]}


def get(key: str) -> Platform:
    try:
        return PLATFORMS[key]
    except KeyError:
        raise KeyError("unknown platform %r; have %s" % (key, sorted(PLATFORMS))) from None


def coverage() -> dict:
    """What the registry can and cannot speak for: how many platforms, how many of them measured
    a hierarchy ratio, the span of those ratios, the number of validation targets."""
    measured = [p.hierarchy_ratio for p in PLATFORMS.values() if p.ratio_measured]
    low, high = min(measured), max(measured)
    return {"n_platforms": len(PLATFORMS), "n_ratio_measured": len(measured),
            "ratio_min": low, "ratio_max": high, "spans_hierarchical": high >= HIERARCHICAL_FROM,
            "targets_total": sum(p.n_targets for p in PLATFORMS.values())}


@dataclass
class Archetype:
    key: str
    label: str
    fast_side: str
    slow_side: str
    ratio_nominal: float
    note: str = ""


def _synthetic(ratio: int) -> Archetype:
    return Archetype("ratio-%d" % ratio, "Synthetic ratio scenario", "synthetic", "synthetic",
                     float(ratio), "Sensitivity point; not assigned to a named platform.")


ARCHETYPES = [Archetype("measured-a", "Platform A measured ratio", "measured fast side",
                        "measured slow side", 1.03, "The only row whose ratio is measured."),
              *map(_synthetic, (2, 4, 9, 18))]


def verdict(ratio: float, breakevens: dict) -> dict:
    """Two-hop pays at a tier exactly when the ratio reaches that tier's break-even."""
    return {tier: not ratio < needed for tier, needed in breakevens.items()}


def platform_map(q: int = 3, tok: int = 4096) -> list:
    from .sweep import CHAIN_SCENARIOS
    from .uncertainty import breakeven_ratio
    needed = {tier: breakeven_ratio(chain, q=q, tok=tok) for tier, chain in CHAIN_SCENARIOS}
    return [dict(archetype=arch, breakevens=needed, verdict=verdict(arch.ratio_nominal, needed))
            for arch in ARCHETYPES]


def _registry_lines() -> list:
    def ratio(p):
        return "%.2f" % p.hierarchy_ratio if p.ratio_measured else "unresolved"

    def fit_err(p):
        return "n/a" if math.isnan(p.fit_median_err) else "%.1f%%" % (100 * p.fit_median_err)
    cols = [Column("key", "%-5s", lambda p: p.key), Column("platform", "%-60s", lambda p: p.label[:60]),
            Column("ratio", "%10s", ratio), Column("fit err", "%9s", fit_err),
            Column("targets", "%8d", lambda p: p.n_targets)]
    return render_table(cols, [PLATFORMS[k] for k in sorted(PLATFORMS)])


def _scenario_lines() -> list:
    rows = platform_map()
    needed = rows[0]["breakevens"]
    cols = [Column("scenario", "%-44s", lambda r: r["archetype"].label[:44]),
            Column("ratio", "%6.2f", lambda r: r["archetype"].ratio_nominal)]
    for tier, be in needed.items():
        cols.append(Column("%s (>= %.2f)" % (tier[:12], be), "%-22s",
                           lambda r, tier=tier: "yes" if r["verdict"][tier] else "no"))
    return render_table(cols, rows)


def main() -> None:
    print("=== measured platforms ===")
    print("\n".join(_registry_lines()))
    c = coverage()
    print("\n%d platforms, %d validation targets; ratio measured on %d platform(s): %.2f-%.2f"
          % (c["n_platforms"], c["targets_total"], c["n_ratio_measured"], c["ratio_min"],
             c["ratio_max"]))
    if not c["spans_hierarchical"]:
        from .hierarchy import CROSS_SUPERNODE_WORLD128_GBPS, loaded_ratio
        boundary = sorted(loaded_ratio(p) for p in CROSS_SUPERNODE_WORLD128_GBPS)
        print("No registered platform has a ratio above %.1f: the synthetic rows below are\n"
              "sensitivities, not predictions.  Two measured ratios exist off this registry\n"
              "(the two supernode boundaries of platform A): %.2f and %.2f."
              % (HIERARCHICAL_FROM, boundary[0], boundary[-1]))
    print("\n=== ratio-only sensitivity scenarios ===")
    print("\n".join(_scenario_lines()))
    print("\nThese are ratio-only sensitivity scenarios, not deployment verdicts.")


if __name__ == "__main__":
    main()
