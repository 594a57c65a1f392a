"""Numbers quoted in docs/ are recomputed from the module that owns them.

A claim names a document, the sentence the numbers sit in (``{n}`` where each number goes;
whitespace is collapsed before matching) and a function returning the live values.  Editing the
prose or the code alone turns the test red.  Only DERIVED numbers belong here; measured constants
are pinned beside their provenance in tests/test_sim.py.
"""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NUM = r"([-+]?\d+(?:\.\d+)?)"


def _read(rel):
    with open(os.path.join(ROOT, rel), encoding="utf-8") as fh:
        return re.sub(r"\s+", " ", fh.read())


def _numbers(rel, template):
    parts = re.sub(r"\s+", " ", template).split("{n}")
    pattern = re.compile(NUM.join(re.escape(p) for p in parts))
    m = pattern.search(_read(rel))
    assert m, f"sentence not found in {rel}: {template!r}"
    return [float(g) for g in m.groups()]


def _breakevens():
    from terracemoe_simulator_b200.sim import sweep, uncertainty
    return [uncertainty.breakeven_ratio(c) for _, c in sweep.CHAIN_SCENARIOS]


def _width_sweep():
    from terracemoe_simulator_b200.sim import uncertainty
    return [b for _, b in uncertainty.breakeven_vs_hidden_width()]


def _tier1():
    from terracemoe_simulator_b200.sim import calibrate, validate_micro
    _, d = validate_micro.validate_micro(calibrate.flat_supernode(), verbose=False)
    return [100 * d["median"], 100 * d["worst"]]


def _tier1b():
    from terracemoe_simulator_b200.sim import calibrate, validate_sweep as vs
    out = []
    for cluster, targets in ((calibrate.flat_supernode(), vs.TARGETS_A),
                             (calibrate.second_machine(), vs.TARGETS_B),
                             (calibrate.flat_supernode(), vs.TARGETS_C),
                             (calibrate.flat_supernode(), vs.TARGETS_D)):
        out.append(100 * vs.validate_sweep(cluster, targets, verbose=False)[1]["median"])
    return out


def _tier2_mae():
    from terracemoe_simulator_b200.sim import calibrate, validate
    return [validate.validate(calibrate.aug_flat(), verbose=False)[1]["mae"]]


def _overlap():
    from terracemoe_simulator_b200.sim import calibrate, overlap
    res = overlap.evaluate(calibrate.flat_supernode(), verbose=False)
    return [res[k]["mae"] for k in ("M0", "M1", "M2", "M3", "M4", "M5")]


def _m_table():
    from terracemoe_simulator_b200.sim import codesign
    out = []
    for _, _, chain, fused in codesign.m_table():
        out += [chain, fused]
    return out


def _b200_gate():
    from terracemoe_simulator_b200.sim import validate_b200
    _, d = validate_b200.validate_b200(verbose=False)
    return [100 * d["median"], 100 * d["worst"]]


def _b200_constants():
    from terracemoe_simulator_b200.sim import calibrate as c
    return [1e3 * c.B200_ALPHA_ONE_HOP_MS, 1e3 * c.B200_ALPHA_TWO_HOP_MS, c.B200_BETA_GBPS,
            c.B200_SELF_COPY_GBPS / 1e3]


def _b200_grouping_ratios():
    from terracemoe_simulator_b200.sim import calibrate
    rows = {r["R"]: r for r in calibrate.load_b200_sweep() if r["q"] == 3 and r["tokens"] == 16384}
    return [rows[R]["two_hop_ms"] / rows[R]["one_hop_ms"] for R in (1, 2, 4)]


def _phase_spans():
    from terracemoe_simulator_b200.sim import calibrate, core, phase
    g = core.MoEGeometry(name="n4", n_groups=4, R=8, k=6, M=2, seq=4096, mbs=1, gbs=4 * 8 * 4096)
    r = phase.report(calibrate.flat_supernode(), g, {"n_experts": 128, "d_expert": 2048})
    s = r["spans"]
    return [s.splits_sync, s.hop_a, s.arrival_chain, s.hop_b, s.combine]


def _launch_row(tier):
    from terracemoe_simulator_b200.sim import core, profile, sweep
    g = core.MoEGeometry("launch", 16, 8, 6, 2)
    rows = profile.launch_sensitivity(g, sweep.CHAIN_SCENARIOS[tier][1],
                                      deltas_ms=(0.0, 0.04, 0.08, 0.111, 0.16, 0.25))
    return [r["breakeven"] for r in rows]


def _byte_criterion(q):
    from terracemoe_simulator_b200.tools.breakeven import breakeven
    return [breakeven(q, 8), breakeven(q, 8, True, 4), breakeven(q, 2), breakeven(q, 128)]


def _b200_step_worst():
    from terracemoe_simulator_b200.sim import b200_step
    return [100 * b200_step.validate(verbose=False)[1]["worst"]]


CLAIMS = [
    ("docs/05-simulator.md", "the worst error is {n} %", _b200_step_worst, 0.06),
    ("docs/03-applicability.md", "2.49 with the PyTorch arrival chain, 1.49 with the fused-kernel "
     "target and 1.10 with zero implementation overhead".replace("2.49", "{n}", 1)
     .replace("1.49", "{n}", 1).replace("1.10", "{n}", 1), _breakevens, 0.015),
    ("docs/05-simulator.md", "{n} / {n} / {n} for the three arrival-chain tiers", _breakevens, 0.015),
    ("docs/05-simulator.md", "1024 / 2048 / 4096 / 8192: {n} / {n} / {n} / {n}.", _width_sweep, 0.015),
    ("docs/05-simulator.md", "median error {n} %, worst {n} %, crossover", _tier1, 0.06),
    ("docs/05-simulator.md", "three corpora: {n} %, {n} %, {n} % — pass; a fourth corpus measured "
     "through the drift probe fails at {n} %", _tier1b, 0.06),
    ("docs/05-simulator.md", "**fails** (mean error {n},", _tier2_mae, 0.001),
    ("docs/05-simulator.md", "median error {n} %, worst {n} % (`python", _b200_gate, 0.06),
    ("docs/05-simulator.md", "alpha {n} us for the fused one-hop call and {n} us for the two-hop "
     "call, beta {n} GB/s per GPU", lambda: _b200_constants()[:3], 0.06),
    ("docs/05-simulator.md", "local copy at {n} TB/s", lambda: _b200_constants()[3:], 0.006),
    ("docs/07-tier2-overlap.md", "| M0 | no overlap | {n} |", lambda: _overlap()[:1], 0.0006),
    ("docs/07-tier2-overlap.md", "| M1 | proportional | {n} |", lambda: _overlap()[1:2], 0.0006),
    ("docs/07-tier2-overlap.md", "| M3 | hidden fixed cost | {n} |", lambda: _overlap()[3:4], 0.0006),
    ("docs/07-tier2-overlap.md", "| M5 | exposed per micro-batch | {n} |", lambda: _overlap()[5:6],
     0.0006),
    ("docs/12-group-cap.md", "| 4 | 2 | {n} | {n} | | 2 | 4 | {n} | {n} | | 1 | 8 | {n} | {n} |",
     _m_table, 0.0006),
    ("docs/03-applicability.md", "| {n} | | groups of 2 GPUs | {n} | | groups of 4 GPUs | {n} |",
     _b200_grouping_ratios, 0.006),
    ("docs/09-phase-model.md", "the spans are {n} / {n} / {n} / {n} / {n} ms", _phase_spans, 0.0006),
    ("docs/03-applicability.md", "| 2 | {n} | {n} | {n} | {n} |", lambda: _byte_criterion(2), 0.0006),
    ("docs/03-applicability.md", "| 3 | {n} | {n} | {n} | {n} |", lambda: _byte_criterion(3), 0.0006),
    ("docs/03-applicability.md", "| 4 | {n} | {n} | {n} | {n} |", lambda: _byte_criterion(4), 0.0006),
    ("docs/03-applicability.md", "| 6 | {n} | {n} | {n} | {n} |", lambda: _byte_criterion(6), 0.0006),
    ("docs/09-phase-model.md", "| breakeven, PyTorch chain | {n} | {n} | {n} | {n} | {n} | {n} |",
     lambda: _launch_row(0), 0.006),
    ("docs/09-phase-model.md", "| breakeven, fused target | {n} | {n} | {n} | {n} | {n} | {n} |",
     lambda: _launch_row(1), 0.006),
    ("docs/09-phase-model.md", "| breakeven, zero overhead | {n} | {n} | {n} | {n} | {n} | {n} |",
     lambda: _launch_row(2), 0.006),
]


@pytest.mark.parametrize("rel,template,live,tol", CLAIMS,
                         ids=[f"{c[0].split('/')[-1]}:{i}" for i, c in enumerate(CLAIMS)])
def test_quoted_number_matches_the_code(rel, template, live, tol):
    quoted = _numbers(rel, template)
    values = list(live())
    assert len(quoted) == len(values), (quoted, values)
    for q, v in zip(quoted, values):
        assert abs(q - v) <= tol, f"{rel}: prose says {q}, code says {v:.4f}"


def test_every_doc_names_only_existing_files():
    """Paths in backticks that look like repository files must exist."""
    missing = []
    for name in sorted(os.listdir(os.path.join(ROOT, "docs"))):
        if not name.endswith(".md"):
            continue
        text = open(os.path.join(ROOT, "docs", name), encoding="utf-8").read()
        for path in re.findall(r"`([\w./-]+\.(?:py|cu|cuh|h|md|json))`", text):
            cands = [path, os.path.join("terracemoe_simulator_b200", path)]
            if not any(os.path.exists(os.path.join(ROOT, c)) for c in cands):
                missing.append((name, path))
    assert not missing, missing


def test_troute_explainer_example_is_what_the_code_routes():
    """The one-token table of docs/10-troute.md, recomputed by ``t_route``."""
    import torch
    from terracemoe_simulator_b200.routing import TRouteConfig, t_route
    text = _read("docs/10-troute.md")
    aff = torch.tensor([[0.90, 0.85, 0.80, 0.78, 0.30, 0.20, 0.75, 0.72, 0.10, 0.60, 0.15, 0.05]])
    cfg = TRouteConfig(12, 4, 4, 2)
    for mode in ("global_topk", "group_limited", "quota_only", "full"):
        idx, gates, _ = t_route(aff, torch.zeros(12), cfg, mode=mode)
        order = torch.argsort(idx[0])
        experts = " ".join(str(int(e)) for e in idx[0][order])
        groups = ", ".join(str(g) for g in sorted(set((idx[0] // 3).tolist())))
        g = " ".join("%.3f" % v for v in gates[0][order].tolist())
        row = f"| `{mode}` | {experts} | {groups} | {g} |"
        assert row in text, row


def test_troute_explainer_conjunction_share():
    from terracemoe_simulator_b200.tools import route_results as rr
    text = _read("docs/10-troute.md")
    assert "cost %d %% of what the quota alone costs" % round(100 * rr.conjunction_cost_share("20k")) in text
    assert "%d %% at 30 k" % round(100 * rr.conjunction_cost_share("30k")) in text


def test_onesided_doc_quotes_the_sweep():
    import statistics
    from terracemoe_simulator_b200.sim import calibrate
    r = [x["nccl_a2a_x2_ms"] / x["one_hop_ms"] for x in calibrate.load_b200_sweep()
         if x["tokens"] >= 4096]
    lo, med, hi = min(r), statistics.median(r), max(r)
    text = _read("docs/08-onesided.md")
    assert "win by %d-%d %% (median %d %%)" % (round(100 * (lo - 1)), round(100 * (hi - 1)),
                                               round(100 * (med - 1))) in text


def test_profile_summary_quotes_the_roofline_module():
    from terracemoe_simulator_b200.sim import b200_roofline as br
    big = [t for t in br.table() if t["tokens"] == 16384]
    text = _read("profiles/fused_dispatch_combine_8gpu.md")
    want = "reaches %.2f-%.2f of the 770 GB/s roofline and NCCL %.2f-%.2f" % (
        min(t["one_hop_frac"] for t in big), max(t["one_hop_frac"] for t in big),
        min(t["nccl_frac"] for t in big), max(t["nccl_frac"] for t in big))
    assert want in text, want


def test_readme_layer_table_quotes_the_committed_bench_runs():
    """The measured table of the README is the fastest arm of every committed bench run."""
    from terracemoe_simulator_b200.sim import b200_step
    text = _read("README.md")
    for run in b200_step.load_bench()["runs"]:
        best = min(run["paths"].values())
        n = run["n_gpus"]
        if n == 1:
            assert "| 1 GPU | 25.6 ms | 3.47-3.57 ms |" in text and 3.47 <= round(best, 2) <= 3.57
        else:
            assert "| %d GPUs |" % n in text and "%.2f ms" % best in text, (n, best)
    doc = _read("docs/14-overlap-plan.md")
    steps = b200_step.measured_steps()
    for n, rpn in ((2, 1), (4, 1), (8, 2)):
        cells = [steps[n, rpn, p, s] for p, s in (("one_hop", "overlap"), ("one_hop", "serial"),
                                                  ("two_hop", "overlap"), ("two_hop", "serial"))]
        for v in cells:
            assert "%.2f" % v in doc, (n, v)
