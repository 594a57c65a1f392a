"""Cost-model contracts: ledgers, gates (including the pinned NEGATIVE results), snapshots."""
import dataclasses
import math

import pytest

from terracemoe_simulator_b200 import sim
from terracemoe_simulator_b200.sim import (archsearch, calibrate, chain_remeasured, codesign,
                                           compute, core, envelope, fit, hierarchy, hostregime,
                                           imbalance, machine, overlap, phase, platforms, profile,
                                           record, sweep, tiers, twohop_measured, uncertainty,
                                           validate, validate_b200, validate_micro, validate_sweep)
from terracemoe_simulator_b200.tools import breakeven as be_cli

FLAG = core.MoEGeometry("flag", 16, 8, 6, 2)


def test_lazy_exports():
    assert sim.ClusterSpec is core.ClusterSpec and sim.MoEGeometry is core.MoEGeometry
    assert sim.one_hop_call is core.one_hop_call and len(sim.HOLDOUTS) == 7
    with pytest.raises(AttributeError):
        sim.no_such_name


def test_geometry_ledger():
    assert FLAG.q == 3 and FLAG.ep == 128 and FLAG.tokens_per_rank == 4096
    assert FLAG.microbatches == 4
    assert FLAG.calls_per_step_fwd() == 152 and FLAG.calls_per_step_bwd() == 76
    assert FLAG.rows_one_hop() == 24576 and FLAG.rows_hop_a() == 8192 and FLAG.rows_hop_b() == 24576
    assert FLAG.row_bytes() == 4096
    assert core.step_delta(calibrate.flat_supernode(), FLAG)["calls_per_step"] == 456
    with pytest.raises(ValueError):
        core.MoEGeometry("bad", 16, 8, 6, 4).q
    with pytest.raises(ValueError):
        core.MoEGeometry("bad", 16, 8, 6, 2, gbs=100).microbatches


def test_hop_a_self_fraction_and_interp():
    assert core.hop_a_self_fraction(FLAG) == 1.0 / 16
    assert core.hop_a_self_fraction(core.MoEGeometry("one", 1, 8, 6, 2)) == 1.0
    lvl = core.Level("x", [(2, 1.0), (4, 3.0)], [(10.0, 1.0), (1000.0, 3.0)])
    assert lvl.alpha_ms(1) == 1.0 and lvl.alpha_ms(3) == 2.0 and lvl.alpha_ms(9) == 3.0
    assert math.isclose(lvl.beta_gbps(100.0), 2.0)
    with pytest.raises(ValueError):
        core.Level("empty").alpha_ms(2)


def test_two_hop_is_sum_of_parts_and_overlap_knob():
    c = calibrate.flat_supernode()
    p = core.two_hop_parts(c, FLAG)
    assert math.isclose(core.two_hop_call(c, FLAG), sum(p.values()))
    assert math.isclose(p["chain"], 1.042, rel_tol=1e-3) and p["splits"] == 0.044
    full = dataclasses.replace(c, hop_overlap=1.0)
    assert math.isclose(core.two_hop_call(c, FLAG) - core.two_hop_call(full, FLAG),
                        min(p["hop_a"], p["hop_b"]))


def test_tier1_passes_with_pinned_numbers():
    ok, d = validate_micro.validate_micro(calibrate.flat_supernode(), verbose=False)
    assert ok and abs(d["median"] - 0.041) < 0.002 and abs(d["worst"] - 0.245) < 0.002
    assert d["cross"] == (4096, 8192)


def test_tier2_must_fail():
    ok, d = validate.validate(calibrate.aug_flat(), verbose=False)
    assert not ok                      # pinned negative result: step-level extrapolation locked
    assert abs(d["mae"] - 0.1353) < 0.002 and d["in_tol"] == 0


def test_overlap_families_all_fail_with_pinned_mae():
    res = overlap.evaluate(calibrate.flat_supernode(), verbose=False)
    want = {"M0": 0.048, "M1": 0.153, "M2": 0.080, "M3": 0.133, "M4": 0.080, "M5": 0.108}
    for key, mae in want.items():
        assert not res[key]["gate"] and abs(res[key]["mae"] - mae) < 0.005


def test_tier1b_corpora():
    a = validate_sweep.validate_sweep(calibrate.flat_supernode(), validate_sweep.TARGETS_A, verbose=False)
    b = validate_sweep.validate_sweep(calibrate.second_machine(), validate_sweep.TARGETS_B, verbose=False)
    c = validate_sweep.validate_sweep(calibrate.flat_supernode(), validate_sweep.TARGETS_C, verbose=False)
    d = validate_sweep.validate_sweep(calibrate.flat_supernode(), validate_sweep.TARGETS_D, verbose=False)
    assert a[0] and b[0] and c[0] and not d[0]
    assert abs(a[1]["median"] - 0.019) < 0.002 and abs(b[1]["median"] - 0.093) < 0.002
    assert abs(c[1]["median"] - 0.080) < 0.002 and abs(d[1]["median"] - 0.151) < 0.002
    assert len(validate_sweep.TARGETS_A) == 6 and len(validate_sweep.TARGETS_B) == 44
    # adopting the measured alpha(8) clears corpus D
    fixed = calibrate.flat_supernode()
    fixed.flat.alpha_pts = [(2, 0.09), (8, 0.129)] + fixed.flat.alpha_pts[2:]
    assert validate_sweep.validate_sweep(fixed, validate_sweep.TARGETS_D, verbose=False)[0]


def test_breakeven_snapshots_and_bands():
    got = [uncertainty.breakeven_ratio(c) for _, c in sweep.CHAIN_SCENARIOS]
    for g, want in zip(got, (2.49, 1.49, 1.10)):
        assert abs(g - want) < 0.02
    assert uncertainty.mc_band(3.2, 0.012) == uncertainty.mc_band(3.2, 0.012)   # reproducible
    p5, med, p95 = uncertainty.mc_band(1.03, calibrate.CHAIN_US_PER_ROW)
    assert p5 <= med <= p95 and p95 <= 1.0          # flat machine with the chain: never wins
    assert uncertainty.mc_band(8.0, calibrate.CHAIN_US_PER_ROW)[0] > 1.0
    widths = dict(uncertainty.breakeven_vs_hidden_width())
    for H, want in ((1024, 3.37), (2048, 2.49), (4096, 2.02), (8192, 1.80)):
        assert abs(widths[H] - want) < 0.02


def test_heatmap_monotone_and_geometry_grid():
    grid, ratios, toks = uncertainty.heatmap(0.012)
    for row in grid:
        assert all(b >= a - 1e-9 for a, b in zip(row, row[1:]))
    rows = uncertainty.geometry_grid(0.012)
    assert len(rows) == 54 and all(1.0 <= r[4] <= 3.0 for r in rows)
    lo, hi = uncertainty.scale_band(512)
    assert hi / lo > 1.8


def test_sweep_table_shape():
    table = sweep.ratio_table()
    for name, tier in table.items():
        for q, cells in tier.items():
            if "upper bound" not in name:
                assert cells[0] <= 1.0                          # ratio 1.03 column
            assert all(b >= a for a, b in zip(cells, cells[1:]))
    fused = table["hypothetical fused target"][3]
    assert abs(fused[0] - 0.81) < 0.02 and abs(fused[2] - 1.51) < 0.02


def test_calibration_identities():
    assert abs(calibrate.PER_PEER_MESSAGE_US - 0.469) < 0.002
    tab = calibrate.saturating_beta(100.0, 54 * 1024)
    assert tab[0][0] <= 1.0 and abs(tab[-1][1] - 100.0) < 0.1
    assert all(b2 >= b1 for (_, b1), (_, b2) in zip(tab, tab[1:]))
    assert calibrate.saturating_beta(80.0, 0.0)[3][1] == 80.0
    syn = calibrate.synthetic(4.0)
    assert abs(syn.ratio() - 4.0) < 0.05 and abs(calibrate.flat_supernode().ratio() - 1.03) < 0.06
    assert calibrate.aug_flat is calibrate.flat_supernode


def test_profile_checklist_never_contradicts_model():
    g = core.MoEGeometry("op", 16, 8, 6, 2, seq=4096, mbs=1, gbs=16 * 8 * 4096)
    for spec, ratio in ((calibrate.flat_supernode(), None), (calibrate.synthetic(9.0), 9.0),
                        (calibrate.synthetic(9.0, chain_us_per_row=0.012), 9.0)):
        r = profile.profile_from_spec(spec, g, ratio)
        assert len(r["conditions"]) == 6
        if r["verdict"]["qualifies"]:
            assert r["model_ratio"] > 1.0
    assert not profile.profile_from_spec(calibrate.flat_supernode(), g)["verdict"]["qualifies"]
    assert profile.byte_breakeven(8, 3) == pytest.approx(1.3125)
    assert profile.byte_breakeven(8, 1) == float("inf")
    unknown = profile.check(9.0, 8, 6, 2, 128, 4096, 2048, 0.012, alpha_of_world=None)
    assert "UNKNOWN" in unknown[4].detail and not unknown[4].passed
    sens = profile.bandwidth_world_sensitivity()
    for (_, _, per_world), want in zip(sens, (2.88, 1.78, 1.34)):
        assert abs(per_world - want) < 0.03
    ls = profile.launch_sensitivity(g, 0.012)
    assert all(b["breakeven"] >= a["breakeven"] for a, b in zip(ls, ls[1:]))


def test_breakeven_cli_closed_form_agrees_with_profile():
    for R in (2, 4, 8):
        for q in (2, 3, 6):
            assert be_cli.breakeven(q, R) == pytest.approx(profile.byte_breakeven(R, q))
    assert be_cli.breakeven(3, 8, dedup=True) < be_cli.breakeven(3, 8)
    assert be_cli.D_of(1, 8, 4) == pytest.approx(1.0) and be_cli.D_of(0, 8, 4) == 0.0


def test_machine_and_compute():
    assert abs(machine.INDEX_NS_PER_ROW - 28.6) < 0.1 and abs(machine.GATHER_GBPS_MEASURED - 1469) < 2
    assert abs(machine.chain_us_per_row_at(2048) - 0.0424) < 1e-4
    with pytest.raises(ValueError):
        machine.chain_us_per_row_at(3000)
    with pytest.raises(ValueError):
        machine.Accelerator("x", 100.0, 10.0, 0.1).gather_gbps
    acc = machine.ASCEND_910C
    assert machine.PYTORCH_CHAIN.ms(73728, 2048, acc) == pytest.approx(2.51, rel=0.03)
    assert machine.NO_CHAIN.ms(10 ** 6, 4096, acc) == 0.0
    assert machine.FUSED_CHAIN.ms(10, 2048, acc) == acc.launch_ms
    model = machine.MoEModel("m", 4096, 64)
    assert machine.min_expert_parallelism(model, machine.B200, 0.2) >= 1
    assert machine.spans_multiple_domains(16, 8) and not machine.spans_multiple_domains(8, 8)
    assert compute.achieved_tflops(4096) == 327.4 and compute.achieved_tflops(100) == 141.6
    r = compute.expert_ffn(4096, 6, 128, 128, 2048, 2048)
    assert r["rows_per_expert"] == 24576 and r["ms_lo"] < r["ms"] < r["ms_hi"]
    assert compute.expert_ffn_b200(4096, 6, 64, 8, 4096, 1408)["tflops"] > 1000
    assert compute.comm_share_upper_bound(1.0, 3.0) == 0.25


def test_imbalance_kept_out_of_core():
    import inspect
    assert "imbalance" not in inspect.getsource(core)
    f = imbalance.strategy_inflation(128, 16, 8, 3)
    assert f["one_hop"] > f["hop_b"] > 1.0 and f["one_hop"] > f["hop_a"]
    out = imbalance.adjusted_ratio(calibrate.synthetic(3.2, chain_us_per_row=0.012), FLAG)
    assert out["shift"] > 0


def test_codesign_envelope_archsearch_record():
    rows = codesign.m_table()
    for (M, q, g_chain, g_fused), want in zip(rows, ((1.362, 1.649), (1.960, 2.614), (2.510, 3.694))):
        assert abs(g_chain - want[0]) < 0.005 and abs(g_fused - want[1]) < 0.005
    with pytest.raises(ValueError):
        codesign.MoEArch("x", 64, 64, 8, 6, M=4).q
    m = codesign.synthetic_dgx_h100()
    prof = codesign.profile(codesign.REFERENCE_ARCH, m)
    assert prof["binds"] in ("memory capacity", "expert matmul, memory bound",
                             "expert matmul, compute bound") and prof["memory_caveat"]
    assert m.fabric.fixed_cost_condition()["clears"]
    d = codesign.dispatch_breakdown(codesign.REFERENCE_ARCH, codesign.hgx_b200())
    assert d["ep"] == 8 and d["chain_ms"] == 0.0
    env = envelope.envelope(codesign.REFERENCE_ARCH, m)
    assert len(env["points"]) == 9 and "band on 128 accelerators" in envelope.table(env)
    assert envelope.first_order_threshold(m) == pytest.approx(989e12 / (3 * 50e9))
    cands = archsearch.search(codesign.REFERENCE_ARCH, m)
    assert cands and archsearch.rank(cands)[0].no_overlap_ms <= archsearch.rank(cands)[-1].no_overlap_ms
    assert all(record.checks().values())


def test_phase_refuses_to_extrapolate():
    r = phase.report(calibrate.flat_supernode(), FLAG, {"n_experts": 128, "d_expert": 2048})
    assert not r["calibrated"] and len(r["missing"]) == 3
    with pytest.raises(NotImplementedError):
        phase.step_ms(r["spans"], phase.OverlapModel(), 4, 19)
    full = phase.OverlapModel(0.5, 100.0, True)
    assert phase.step_ms(r["spans"], full, 4, 19) > 0


def test_measurement_records():
    assert twohop_measured.every_configuration_wins()
    gs = [twohop_measured.g(r) for r in twohop_measured.MEASURED]
    assert abs(gs[0] - 1.77) < 0.01 and abs(gs[2] - 2.23) < 0.01 and abs(gs[1] - 1.43) < 0.01
    assert 0.2 < twohop_measured.chain_share(twohop_measured.MEASURED[0]) < 0.3
    assert len(hostregime.MEASURED) == 46
    assert abs(hostregime.plateau("burst", 8) - 0.1217) < 0.001
    assert abs(hostregime.plateau("percall", 16) - 0.2933) < 0.001
    with pytest.raises(ValueError):
        hostregime.rows("hourly")
    assert abs(hierarchy.hierarchy_ratio("percall") - 2.55) < 0.02
    assert abs(hierarchy.hierarchy_ratio("burst") - 2.58) < 0.02
    assert abs(hierarchy.loaded_ratio("pool110/pool111") - 5.10) < 0.01
    assert abs(hierarchy.loaded_ratio("pool110/pool12") - 7.51) < 0.01
    place = hierarchy.placement()
    assert all(place["clears"].values())
    assert 0 < place["ratio"] - place["thresholds"]["PyTorch chain (measured)"] < 0.1
    assert tiers.peer_counts(tiers.Topology(), 128, 8) == {"intra_node": 7, "cross_node": 56,
                                                           "cross_supernode": 64}
    assert tiers.peer_effect_span() < 1.10
    with pytest.raises(ValueError):
        tiers.tier_at("cross_supernode", 3)
    assert chain_remeasured.published_sweep_is_at_pairs()
    assert abs(chain_remeasured.us_per_row_here() - 0.0291) < 0.0005
    maes = [v[0] for v in chain_remeasured.chain_cancels_in_validation().values()]
    assert max(maes) - min(maes) < 1e-9


def test_fit_recovers_constants_and_marginal_bandwidth():
    pytest.importorskip("scipy")
    recs = [("syn", w, float(s), fit.predict_ms(w, s, 0.3, 118.0, 320 * 1024))
            for s in (2 ** 20, 2 ** 22, 2 ** 24, 2 ** 26, 2 ** 28) for w in (8, 16, 128)]
    free = fit.fit_frame(recs)
    assert abs(free["beta_inf"] - 118.0) < 3 and free["median_rel_err"] < 1e-3
    pinned = fit.fit_beta_pinned(recs, lambda w: 0.3)
    assert abs(pinned["x_half"] / (320 * 1024) - 1) < 0.05
    mb = fit.marginal_bandwidth([(w, s, ms) for _, w, s, ms in recs])
    assert abs(mb[128] - 118.0) < 3
    forms = fit.compare_forms(recs, exponents=(1.0, 2.0))
    assert set(forms) == {"additive (shipped)", "quadrature"}
    under = fit.fit_pinned_under_form(recs, lambda w: 0.3, p=1.0)
    assert under["beta_inf"] > 50
    assert fit.audit(recs, verbose=False)["syn"]["n"] == 15
    dict_recs = [{"frame": "flat", "world": w, "bytes": s, "ms": ms} for _, w, s, ms in recs]
    assert len(fit._norm(dict_recs)) == 15


def test_b200_platform_and_gate():
    ok, d = validate_b200.validate_b200(verbose=False)
    assert d["median"] < 0.10                                   # in-sample: fit quality
    # one 256-token row of the sweep was caught at twice its neighbours' time and stays in the
    # data; the robust fit ignores it, the score shows it
    far = [r for r in d["in_sample"]["rows"] if abs(r[9]) > 0.15]
    assert len(far) <= 1 and all(r[2] == 256 for r in far)
    held = d["holdout"]                                         # prediction: rows the fit never saw
    train, rest = validate_b200.split_holdout(calibrate.load_b200_sweep())
    assert held["n"] == len(rest) and len(train) + len(rest) == 48
    assert all(r["R"] in (1, 4) and r["tokens"] <= 4096 for r in train)
    assert held["median"] < 0.10
    predictions = [held] + list(d["cross_size"].values())
    assert ok == all(s["median"] <= 0.10 for s in predictions)
    assert d["every_row"] == all(s["worst"] <= 0.10 for s in predictions)
    assert len(d["beyond"]) == sum(len(validate_b200.beyond(s)) for s in predictions)
    assert all(abs(e) > 0.10 for _r, _q, _t, e in d["beyond"])
    rows = calibrate.load_b200_sweep()
    assert len(rows) == 48 and {r["R"] for r in rows} == {1, 2, 4}
    pytest.importorskip("scipy")
    fitted = calibrate.b200_from_sweep(rows)
    assert abs(fitted.flat.beta_gbps(1e6) - calibrate.B200_BETA_GBPS) < 30
    assert abs(fitted.self_copy_gbps - calibrate.B200_SELF_COPY_GBPS) < 200
    # Hop B inside one GPU waits for no peer: its fixed cost is the smaller one, shipped and fitted
    assert fitted.fast.alpha_ms(1) < fitted.fast.alpha_ms(2) == fitted.fast.alpha_ms(8)
    assert calibrate.B200_ALPHA_FAST_LOCAL_MS < calibrate.B200_ALPHA_FAST_MS
    only_r1 = calibrate.b200_from_sweep([r for r in rows if r["R"] == 1])
    assert only_r1.fast.alpha_ms(1) == only_r1.fast.alpha_ms(4)      # remote cost unseen: tied
    assert platforms.get("B200").hierarchy_ratio == 1.0 and platforms.coverage()["n_platforms"] == 3
    # the registry's B200 line is the live gate: same target count, same median error
    from terracemoe_simulator_b200.sim import calibrate as _cal, validate_b200 as _vb
    _, d = _vb.validate_b200(verbose=False)
    b = platforms.get("B200")
    assert b.n_targets == len(_cal.load_b200_sweep()) and abs(b.fit_median_err - d["median"]) < 1e-3
    with pytest.raises(KeyError):
        platforms.get("Z")
    # token-level dedup (groups of one GPU) is where two-hop pays on a flat NVSwitch
    c = calibrate.b200_nvswitch()
    g1 = core.MoEGeometry("r1", 8, 1, 6, 2, H=4096, seq=4096, gbs=8 * 4096)
    g2 = core.MoEGeometry("r2", 4, 2, 6, 2, H=4096, seq=4096, gbs=8 * 4096)
    assert core.two_hop_call(c, g1) < core.one_hop_call(c, g1)
    assert core.two_hop_call(c, g2) > 0.9 * core.one_hop_call(c, g2)


def test_b200_step_model_within_gate():
    """Both schedules of the layer step, every measured (GPUs, path): the model stays inside
    the gate, and no measured number lives in the module's source."""
    from terracemoe_simulator_b200.sim import b200_step
    bench = b200_step.load_bench()
    steps = b200_step.measured_steps(bench)
    assert {k[3] for k in steps} == {"serial", "overlap"} and (1, 1, "local", "serial") in steps
    ok, d = b200_step.validate(verbose=False)
    assert ok and d["worst"] <= b200_step.GATE and len(d["rows"]) == len(steps) >= 9
    kern = b200_step.kernels(bench)
    g1, g8 = b200_step.gemm_ms(1), b200_step.gemm_ms(8)
    assert g1["tile_efficiency"] < 0.9 < g8["tile_efficiency"] <= 1.0
    assert g1["wgrad_tflops"] == pytest.approx(kern.tflops_wgrad_short, rel=1e-6)
    assert g8["ms"] < g1["ms"] and g1["fwd_ms"] + g1["bwd_ms"] == pytest.approx(g1["ms"])
    # a slower clock stretches the GEMM term and nothing else
    slow = b200_step.gemm_ms(1, sm_mhz=kern.gemm_alone_sm_mhz / 2)
    assert slow["ms"] == pytest.approx(2 ** kern.clock_exponent * g1["ms"])
    # the 8-GPU steps are predictions: the fitted constants never saw them
    assert 8 not in kern.fitted_on_gpus and 0 < d["worst_predicted"] <= b200_step.GATE
    with pytest.raises(ValueError):
        b200_step.predict_ms(2, 1, "one_hop", schedule="pipelined")
    import inspect
    src = inspect.getsource(b200_step)
    assert "MEASURED_MS" not in src and "3.27" not in src and "1300" not in src


def test_b200_step_overlap_term_follows_the_chunked_schedule():
    """What the overlap schedule removes is what ChunkedSchedule says: all of the dispatch but
    the first chunk, the hidden share of the return leg, minus the local reduction; two-hop
    pays its relay on top.  Measured and modelled gains agree in sign for every (GPUs, path)."""
    from terracemoe_simulator_b200.sim import b200_step
    from terracemoe_simulator_b200.sim.phase import ChunkedSchedule
    kern = b200_step.kernels()
    for n, rpn in ((2, 1), (4, 1), (8, 2)):
        serial = b200_step.predict_ms(n, rpn, "one_hop", "serial")
        overlap = b200_step.predict_ms(n, rpn, "one_hop", "overlap")
        one_way = 0.5 * serial["comm_ms"]
        plan = ChunkedSchedule(chunks=2, local_reduce_ms=b200_step.local_reduce_ms(kern),
                               return_hidden=kern.return_hidden)
        g = serial["gemm"]
        want = sum(plan.exposed_ms(one_way, g[part], one_way) for part in ("fwd_ms", "bwd_ms"))
        assert overlap["exposed_ms"] == pytest.approx(want)
        assert serial["gemm_ms"] == overlap["gemm_ms"] and overlap["total_ms"] < serial["total_ms"]
        two = b200_step.predict_ms(n, rpn, "two_hop", "overlap")
        assert two["exposed_ms"] > 2 * kern.two_hop_relay_ms
    for n, rpn, path, measured, model in b200_step.overlap_gain(verbose=False):
        assert (measured > 0) == (model > 0), (n, path, measured, model)
    # more chunks expose less of the dispatch; nothing hides when the GEMM is shorter than a push
    few, many = ChunkedSchedule(chunks=2), ChunkedSchedule(chunks=4)
    assert many.exposed_ms(0.4, 2.0, 0.0) < few.exposed_ms(0.4, 2.0, 0.0)
    assert few.exposed_ms(0.4, 0.1, 0.0) == pytest.approx(0.2 + (0.2 - 0.05) + few.local_reduce_ms)


def test_b200_step_path_ratios_report_the_miss():
    """two-hop / one-hop at step level: the fitted pairs within 3 %, the predicted ones listed
    with their error whatever it is (the 8-GPU overlap pair is the known miss)."""
    from terracemoe_simulator_b200.sim import b200_step
    rows = b200_step.path_ratios(verbose=False)
    assert len(rows) >= 6 and {r[2] for r in rows} == {"serial", "overlap"}
    assert all(abs(r[5]) < 0.03 for r in rows if r[6])
    predicted = [r for r in rows if not r[6]]
    assert predicted and all(r[0] == 8 for r in predicted)
    assert max(abs(r[5]) for r in predicted) < 0.15


def test_b200_step_reads_bench_lines(tmp_path):
    """``--bench FILE`` takes the JSON lines bench.py prints; *_pull paths become serial arms."""
    import json
    from terracemoe_simulator_b200.sim import b200_step
    line = {"impl": "ours", "n_gpus": 2, "config": {"rpn": 1}, "impl_detail": {"chunks": 2, "schedule": "overlap"},
            "paths": {"one_hop": {"ms_per_step": 3.4}, "one_hop_pull": {"ms_per_step": 3.7}}}
    f = tmp_path / "bench.jsonl"
    f.write_text("noise\n" + json.dumps(line) + "\n" + json.dumps({"impl": "reference", "n_gpus": 2}) + "\n")
    bench = b200_step.load_bench(str(f))
    assert b200_step.measured_steps(bench) == {(2, 1, "one_hop", "overlap"): 3.4,
                                               (2, 1, "one_hop", "serial"): 3.7}
    ok, d = b200_step.validate(verbose=False, bench=bench)
    assert len(d["rows"]) == 2


def test_b200_roofline_ledger_and_fractions():
    from terracemoe_simulator_b200.sim import b200_roofline as br
    # the byte ledger of the headline configuration (per GPU and direction)
    one = br.egress_bytes("one_hop", 4096, 6, 2, 4096, 8, 2)
    two = br.egress_bytes("two_hop", 4096, 6, 2, 4096, 8, 2)
    assert one["total"] == pytest.approx(176.2e6, rel=1e-3)
    assert two["hop_a"] == pytest.approx(50.3e6, rel=1e-3) and two["hop_b"] == pytest.approx(100.7e6, rel=1e-3)
    assert br.egress_bytes("two_hop", 4096, 6, 2, 4096, 8, 2, dedup=True)["hop_b"] < two["hop_b"]
    assert br.egress_bytes("two_hop", 4096, 6, 2, 4096, 8, 1)["hop_b"] == 0.0      # groups of one GPU
    with pytest.raises(ValueError):
        br.egress_bytes("three_hop", 1, 2, 1, 8, 8, 2)
    # direction agrees with the closed-form byte criterion at ratio 1: fewer bytes iff q > R
    for R, q, fewer in ((2, 3, True), (8, 3, False), (4, 6, True)):
        a = br.egress_bytes("one_hop", 4096, 2 * q, 2, 2048, 128, R)["total"]
        b = br.egress_bytes("two_hop", 4096, 2 * q, 2, 2048, 128, R)["total"]
        assert (b < a) is fewer
    rows = br.table()
    assert len(rows) == 48
    big = [t for t in rows if t["tokens"] == 16384]
    assert all(0.70 <= t["one_hop_frac"] <= 0.85 for t in big)          # of the measured 770 GB/s
    assert all(t["nccl_frac"] <= t["one_hop_frac"] + 1e-9 for t in big)  # the stores beat NCCL
    assert all(t["one_hop_frac"] < 1.0 and t["two_hop_frac"] < 1.0 for t in rows)
