"""Regenerate every figure from live computations and the recorded measurements.

    python -m terracemoe_simulator_b200.tools.gen_figures [--out docs/figures] [--only f8 f17]

Figures are SVG text written by ``tools/svgplot.py`` (no plotting library is needed), byte-for-byte
reproducible: running twice gives identical files.  The set follows the reference's three
generators (``tools/gen_figures.py``, ``tools/gen_route_figures.py``, ``tools/gen_sim_figures.py``):
published routing results (f1-f6, data in `tools/route_results.py`), cost-model figures computed
live (f7-f11, f13, f16), the one-sided comparison from the B200 sweep (f12), routing
figures computed live from ``routing.t_route`` (f14, f15), plus two figures of this package's own
measurements on 8 x B200 (f19 layer step against its model, f17 measured against modelled two-hop/one-hop ratio, f18 dispatch +
combine time against tokens per GPU).
"""
from __future__ import annotations

import argparse
import os
import sys

from .svgplot import Chart, heatmap

from . import route_results as rr


def f1_loss_axis():
    c = Chart("f1  Loss cost of constrained routing against unconstrained top-k (90 % intervals)",
              "routing mode", "extra loss (nats)", xcats=list(rr.MODES), width=700)
    for i, (readout, color) in enumerate((("20k", "#9ecae1"), ("30k", "#1f77b4"))):
        c.bars([rr.LOSS_COST[readout][m][0] for m in rr.MODES], label="read out at " + readout,
               color=color, group=i, n_groups=2)
    lo, hi = rr.LOSS_COST["20k"]["full"][1:]
    c.note("full at 20k: +%.5f nats [%+.5f, %+.5f]; %.0f %% of what the quota alone costs"
           % (rr.LOSS_COST["20k"]["full"][0], lo, hi, 100 * rr.conjunction_cost_share()))
    return c.render()


def f2_per_seed():
    c = Chart("f2  The same loss differences per seed", "seed", "extra loss (nats)",
              xcats=["seed 1", "seed 2", "seed 3", "seed 4"], width=700)
    for m, color in zip(rr.MODES, ("#2ca02c", "#d62728", "#1f77b4")):
        c.line(range(4), rr.PER_SEED["20k"][m], label=m + " @20k", color=color)
        c.line(range(4), rr.PER_SEED["30k"][m], label=m + " @30k", color=color, dash="4,3")
    c.hline(0.0, None)
    return c.render()


def f3_downstream():
    names = list(rr.DOWNSTREAM_PP)
    c = Chart("f3  Downstream accuracy of T-Route against top-k (percentage points)", "task",
              "difference (pp)", xcats=names)
    c.bars([rr.DOWNSTREAM_PP[n][0] for n in names], color="#1f77b4", label="mean difference")
    c.hline(rr.EQUIVALENCE_PP, "equivalence bounds +-%.1f pp" % rr.EQUIVALENCE_PP, "#d62728")
    c.hline(-rr.EQUIVALENCE_PP, None, "#d62728")
    c.note("90 % intervals: " + "; ".join("%s [%+.3f, %+.3f]" % (n, *rr.DOWNSTREAM_PP[n][1:])
                                          for n in names))
    return c.render()


def f4_load_axis():
    c = Chart("f4  Load balance against top-k: entropy and coefficient of variation", "routing mode",
              "difference", xcats=list(rr.MODES), width=700)
    c.bars([rr.LOAD_ENTROPY[m][0] for m in rr.MODES], label="load entropy", color="#2ca02c",
           group=0, n_groups=2)
    c.bars([rr.LOAD_CV[m][0] for m in rr.MODES], label="load CV", color="#ff7f0e", group=1,
           n_groups=2)
    c.hline(0.0, None)
    return c.render()


def f5_step_neutral():
    c = Chart("f5  Step-time effect of T-Route alone (two runs)", "run", "G = t(top-k) / t(T-Route)",
              xcats=["run 1", "run 2", "mean"])
    mean = sum(rr.STEP_G) / len(rr.STEP_G)
    c.bars(list(rr.STEP_G) + [mean], color="#2ca02c").hline(1.0, "neutral")
    c.ylim = (0.95, 1.03)
    return c.render()


def f6_forerunner():
    names = [m[0] for m in rr.FORERUNNER]
    c = Chart("f6  Small-scale forerunner: hold-out loss of the four modes", "routing mode",
              "hold-out loss", xcats=names, width=700)
    c.bars([m[1] for m in rr.FORERUNNER], color="#1f77b4")
    c.ylim = (6.024, 6.036)
    c.note("load entropy: " + ", ".join("%s %.3f" % (m[0], m[3]) for m in rr.FORERUNNER))
    return c.render()


def f12_onesided():
    from ..sim import calibrate
    rows = sorted((r["tokens"], r["one_hop_ms"], r["nccl_a2a_x2_ms"])
                  for r in calibrate.load_b200_sweep() if r["q"] == 3 and r["R"] == 2)
    c = Chart("f12  One-sided peer-memory stores against the collective, 8 x B200 (there + back)",
              "tokens per GPU", "collective time / one-sided time", xlog=True)
    c.line([r[0] for r in rows], [r[2] / r[1] for r in rows], label="NCCL all-to-all x2 / fused one-hop")
    c.hline(1.15, "criterion 1.15", "#d62728")
    c.hline(1.0, "parity")
    c.note("reference machine: 0.68 (collective wins)")
    return c.render()


def f7_overlap_families():
    from ..sim import calibrate, overlap
    res = overlap.evaluate(calibrate.flat_supernode(), verbose=False)
    keys = sorted(res)
    c = Chart("f7  Step-level overlap families: hold-out error (all fail the gate)",
              "family", "mean |G error|", xcats=keys)
    c.bars([res[k]["mae"] for k in keys], color="#d62728").hline(overlap.GATE_MAE, "gate")
    return c.render()


def f8_breakeven_map():
    from ..sim import uncertainty
    from ..sim.sweep import CHAIN_SCENARIOS
    grid, ratios, toks = uncertainty.heatmap(CHAIN_SCENARIOS[1][1])
    return heatmap(grid, ["%g" % r for r in ratios], [str(t) for t in toks],
                   "f8  one-hop / two-hop time, fused-chain tier, q = 3 (>1: two-hop wins)",
                   "hierarchy ratio (fast / slow bandwidth)", "tokens per rank")


def f9_uncertainty():
    from ..sim import uncertainty
    from ..sim.sweep import CHAIN_SCENARIOS
    ratios = [1.03, 1.5, 2.0, 3.2, 4.5, 8.0, 15.7]
    c = Chart("f9  Monte-Carlo band of the predicted speedup (5th-95th percentile)",
              "hierarchy ratio", "one-hop / two-hop", xlog=True)
    for (name, chain), color in zip(CHAIN_SCENARIOS, ("#d62728", "#1f77b4", "#2ca02c")):
        bands = [uncertainty.mc_band(r, chain) for r in ratios]
        c.band(ratios, [b[0] for b in bands], [b[2] for b in bands], color=color)
        c.line(ratios, [b[1] for b in bands], label=name.split(" (")[0], color=color)
    c.hline(1.0, "breakeven")
    return c.render()


def f10_scale_alpha():
    from ..sim import uncertainty
    curves = uncertainty.scale_treatment_curves()
    worlds = list(uncertainty.EXTRAP_WORLDS)
    c = Chart("f10  Extrapolating alpha(world) past the measured range: four treatments",
              "ranks", "one-hop / two-hop at ratio 3.2", xlog=True)
    for label, ys in curves.items():
        c.line(worlds, ys, label=label.split(" (")[0])
    c.hline(1.0, "breakeven")
    return c.render()


def f11_verdict_bed():
    from ..sim import calibrate, twohop_measured, validate
    ok, d = validate.validate(calibrate.aug_flat(), verbose=False)
    names = [h.geom.name for h in validate.HOLDOUTS]
    c = Chart("f11  Measured end-to-end G on the flat machine (one-hop step / two-hop step)",
              "geometry", "G", xcats=names)
    c.bars([h.g_measured for h in validate.HOLDOUTS], label="measured", color="#1f77b4")
    c.hline(1.0, "neutral")
    c.ylim = (0.8, 1.06)
    c.note("across the supernode boundary the dispatch alone wins: G = " + ", ".join(
        "%.2f" % twohop_measured.g(r) for r in twohop_measured.MEASURED))
    return c.render()


def f13_platform_map():
    from ..sim import platforms
    rows = platforms.platform_map()
    names = [r["archetype"].key for r in rows]
    c = Chart("f13  Where platforms sit against the three breakeven ratios", "platform archetype",
              "hierarchy ratio", xcats=names, ylog=True, width=760)
    c.bars([r["archetype"].ratio_nominal for r in rows], color="#7f7f7f", label="nominal ratio")
    for (tier, be), color in zip(rows[0]["breakevens"].items(), ("#d62728", "#1f77b4", "#2ca02c")):
        c.hline(be, "%s: %.2f" % (tier.split(" (")[0][:22], be), color)
    return c.render()


def f14_routing_modes():
    import torch
    from ..routing import TRouteConfig, t_route
    cfg = TRouteConfig(64, 4, 8, 2)
    aff = torch.rand(4096, 64, generator=torch.Generator().manual_seed(0))
    modes = ["full", "group_limited", "quota_only", "global_topk"]
    groups_touched, max_per_group = [], []
    for m in modes:
        idx, _, _ = t_route(aff, torch.zeros(64), cfg, mode=m)
        grp = idx // cfg.group_size
        onehot = torch.zeros(4096, 4).scatter_add_(1, grp, torch.ones_like(grp, dtype=torch.float))
        groups_touched.append(float((onehot > 0).sum(1).float().mean()))
        max_per_group.append(float(onehot.max(1).values.mean()))
    c = Chart("f14  What each routing mode constrains (64 experts, 4 groups, k=8, M=2)",
              "mode", "per token (mean over 4096 tokens)", xcats=modes, width=700)
    c.bars(groups_touched, label="groups touched", color="#1f77b4", group=0, n_groups=2)
    c.bars(max_per_group, label="largest pick count in one group", color="#ff7f0e", group=1, n_groups=2)
    return c.render()


def f15_routing_costs():
    from ..sim.core import MoEGeometry
    c = Chart("f15  Rows on the wire per rank and collective (4096 tokens, k = 6)", "groups touched M",
              "rows", xcats=["M=1", "M=2", "M=3", "M=6 (top-k)"])
    hop_a, hop_b = [], []
    for M in (1, 2, 3, 6):
        g = MoEGeometry("g", 16, 8, 6, M)
        hop_a.append(g.rows_hop_a())
        hop_b.append(g.rows_hop_b())
    c.bars(hop_a, label="slow level (Hop A)", color="#d62728", group=0, n_groups=2)
    c.bars(hop_b, label="fast level (Hop B) = one-hop rows", color="#1f77b4", group=1, n_groups=2)
    return c.render()


def f16_launch_cost():
    from ..sim import profile
    from ..sim.core import MoEGeometry
    from ..sim.sweep import CHAIN_SCENARIOS
    g = MoEGeometry("op", 16, 8, 6, 2, seq=4096, mbs=1, gbs=16 * 8 * 4096)
    c = Chart("f16  Breakeven ratio against extra launch latency per two-hop call",
              "extra launch latency (ms)", "breakeven hierarchy ratio")
    for name, chain in CHAIN_SCENARIOS:
        ls = profile.launch_sensitivity(g, chain)
        c.line([r["extra_launch_ms"] for r in ls], [min(r["breakeven"], 20.0) for r in ls],
               label=name.split(" (")[0])
    return c.render()


def f17_b200_ratio():
    from ..sim import validate_b200
    ok, d = validate_b200.validate_b200(verbose=False)
    c = Chart("f17  8 x B200: measured against modelled two-hop / one-hop time (fused kernels)",
              "measured ratio", "modelled ratio")
    for R, color in ((1, "#1f77b4"), (2, "#2ca02c"), (4, "#d62728")):
        pts = [(r[7], r[8]) for r in d["rows"] if r[0] == R]
        pts.sort()
        c.line([p[0] for p in pts], [p[1] for p in pts], label="groups of %d GPU%s" % (R, "s"[:R > 1]),
               color=color, dash="1,4")
    lo = min(r[7] for r in d["rows"]); hi = max(r[7] for r in d["rows"])
    c.line([lo, hi], [lo, hi], label="model = measurement", color="#333333", marker=False)
    c.note("median error %.1f%%, worst %.1f%% over %d configurations"
           % (100 * d["median"], 100 * d["worst"], len(d["rows"])))
    return c.render()


def f18_b200_dispatch():
    from ..sim import calibrate
    rows = [r for r in calibrate.load_b200_sweep() if r["q"] == 3]
    c = Chart("f18  8 x B200: fused dispatch + combine time (k = 6, M = 2, H = 4096)",
              "tokens per GPU", "ms (max over ranks)", xlog=True, ylog=True)
    seen = False
    for R, color in ((1, "#1f77b4"), (2, "#2ca02c"), (4, "#d62728")):
        sel = sorted((r["tokens"], r["one_hop_ms"], r["two_hop_ms"], r["nccl_a2a_x2_ms"])
                     for r in rows if r["R"] == R)
        if not sel:
            continue
        if not seen:
            c.line([s[0] for s in sel], [s[1] for s in sel], label="one-hop (fused)", color="#333333")
            c.line([s[0] for s in sel], [s[3] for s in sel], label="NCCL all-to-all x2", color="#999999",
                   dash="4,3")
            seen = True
        c.line([s[0] for s in sel], [s[2] for s in sel], label="two-hop, groups of %d" % R, color=color)
    return c.render()


def f19_b200_step():
    """The layer step on 1-8 GPUs: both schedules, one-hop and two-hop, measured against the
    step model (constants fitted on 1-4 GPUs, 8 GPUs predicted)."""
    from ..sim import b200_step
    bench = b200_step.load_bench()
    steps = b200_step.measured_steps(bench)
    c = Chart("f19  B200: single-MoE-layer step, measured (solid) and modelled (dotted)",
              "GPUs", "ms per step (max over ranks)")
    arms = (("one_hop", "overlap", "#1f77b4"), ("two_hop", "overlap", "#d62728"),
            ("one_hop", "serial", "#7fb2dd"), ("two_hop", "serial", "#eb9a9a"))
    for path, schedule, color in arms:
        pts = sorted((n, rpn, ms) for (n, rpn, p, s), ms in steps.items()
                     if p == path and s == schedule)
        if not pts:
            continue
        xs = [n for n, _rpn, _ms in pts]
        c.line(xs, [ms for _n, _rpn, ms in pts], label="%s, %s" % (path.replace("_", "-"), schedule),
               color=color)
        c.line(xs, [b200_step.predict_ms(n, rpn, path, schedule, bench=bench)["total_ms"]
                    for n, rpn, _ms in pts], label=None, color=color, dash="1,4", marker=False)
    local = steps.get((1, 1, "local", "serial"))
    if local is not None:
        c.note("1 GPU (local kernels): %.2f ms measured, %.2f modelled"
               % (local, b200_step.predict_ms(1, 1, "local", "serial", bench=bench)["total_ms"]))
    return c.render()


FIGURES = {
    "f1-loss-axis": f1_loss_axis, "f2-per-seed": f2_per_seed, "f3-downstream": f3_downstream,
    "f4-load-axis": f4_load_axis, "f5-step-neutral": f5_step_neutral,
    "f6-forerunner": f6_forerunner,
    "f7-overlap-families": f7_overlap_families, "f8-breakeven-map": f8_breakeven_map,
    "f9-uncertainty": f9_uncertainty, "f10-scale-alpha": f10_scale_alpha,
    "f11-verdict-bed": f11_verdict_bed, "f12-onesided": f12_onesided,
    "f13-platform-map": f13_platform_map,
    "f14-routing-modes": f14_routing_modes, "f15-routing-costs": f15_routing_costs,
    "f16-launch-cost": f16_launch_cost, "f17-b200-ratio": f17_b200_ratio,
    "f18-b200-dispatch": f18_b200_dispatch, "f19-b200-step": f19_b200_step,
}


def also_pdf() -> bool:
    """``TERRACE_FIG_PDF=1``: write a vector PDF beside every SVG (off by default)."""
    from ..utils.flags import flag_bool
    return flag_bool("TERRACE_FIG_PDF")


def generate(out_dir: str, only=None, pdf=None) -> list:
    os.makedirs(out_dir, exist_ok=True)
    pdf = also_pdf() if pdf is None else pdf
    written = []
    for name, fn in FIGURES.items():
        if only and not any(name.startswith(o) for o in only):
            continue
        svg = fn()
        path = os.path.join(out_dir, name + ".svg")
        with open(path, "w", encoding="utf-8") as fh:
            fh.write(svg)
        written.append(path)
        if pdf:
            from .svg2pdf import convert
            with open(os.path.join(out_dir, name + ".pdf"), "wb") as fh:
                fh.write(convert(svg))
            written.append(os.path.join(out_dir, name + ".pdf"))
    return written


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--out", default=os.path.join("docs", "figures"))
    ap.add_argument("--only", nargs="*", default=None, help="figure name prefixes, e.g. f8 f17")
    args = ap.parse_args(argv)
    for path in generate(args.out, args.only):
        print("wrote", path)
    return 0


if __name__ == "__main__":
    sys.exit(main())
