"""Probe scripts run under gloo; figure generator is reproducible; one-sided verdict rules."""
import json
import os
import subprocess
import sys
import xml.dom.minidom

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = "terracemoe_simulator_b200"


def _torchrun(nproc, port, module, args):
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", f"{PKG}.bench.{module}"]
    proc = subprocess.run(cmd + args, capture_output=True, env=env, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr.decode(errors="replace")[-3000:]
    return proc.stdout.decode()


def test_a2a_form_probe_both_styles(tmp_path):
    out = tmp_path / "form.json"
    _torchrun(2, 29801, "a2a_form_probe", ["--cpu", "--sizes-mib", "0.0625", "0.25", "--repeats", "2",
                                           "--burst-n", "3", "--percall-n", "3", "--out", str(out)])
    data = json.loads(out.read_text())
    assert data["world"] == 2 and len(data["rows"]) == 2
    assert {r["frame"] for r in data["records"]} == {"burst", "percall"}
    assert all(r["burst_ms"] > 0 and r["percall_ms"] > 0 for r in data["rows"])
    assert set(data["records"][0]) == {"frame", "world", "bytes", "ms"}     # the fitting schema


def test_twohop_verdict_phases(tmp_path):
    out = tmp_path / "verdict.json"
    text = _torchrun(4, 29802, "twohop_verdict", ["--cpu", "--rpn", "2", "--tokens", "64", "--hidden",
                                                  "32", "--repeats", "1", "--calls", "2", "--out",
                                                  str(out)])
    rows = json.loads(out.read_text())["rows"]
    assert [(r["M"], r["q"]) for r in rows] == [(1, 6), (2, 3)]
    for r in rows:
        parts = r["hop_a_ms"] + r["chain_ms"] + r["hop_b_ms"] + r["splits_ms"]
        assert abs(parts - r["two_hop_ms"]) < 1e-9 and r["G"] > 0
    assert "two-hop" in text


def test_fabric_probes(tmp_path):
    a, b = tmp_path / "c.json", tmp_path / "p.json"
    _torchrun(4, 29803, "fabric_contention", ["--cpu", "--sizes-mib", "0.125", "--repeats", "1",
                                              "--calls", "2", "--out", str(a)])
    _torchrun(4, 29804, "fabric_peers", ["--cpu", "--sizes-mib", "0.125", "--repeats", "1",
                                         "--calls", "2", "--out", str(b)])
    cont = json.loads(a.read_text())
    assert [r["active_pairs"] for r in cont["rows"] if r["phase"] == "pairs"] == [1, 2]
    assert cont["rows"][-1]["phase"] == "global" and cont["worst_slowdown"] >= 1.0
    peers = json.loads(b.read_text())
    assert [r["peers"] for r in peers["rows"] if r["phase"] == "peers"] == [1, 2]


def test_peer_splits_are_a_permutation():
    from terracemoe_simulator_b200.bench.fabric_peers import peer_splits
    world, n, chunk = 8, 3, 5
    send = [peer_splits(r, world, n, chunk)[0] for r in range(world)]
    recv = [peer_splits(r, world, n, chunk)[1] for r in range(world)]
    for r in range(world):
        assert sum(send[r]) == n * chunk == sum(recv[r])
        assert all(send[r][p] == 0 for p in range(world) if (p < 4) == (r < 4))   # only across
        for p in range(world):
            assert send[r][p] == recv[p][r]


def test_chain_probes_on_cpu(tmp_path):
    from terracemoe_simulator_b200.bench import chain_live_vs_ref, chain_sweep
    assert chain_live_vs_ref.main(["--tokens", "64", "--hidden", "32", "--calls", "2", "--cpu"]) == 0
    out = tmp_path / "chain.json"
    assert chain_sweep.main(["--out", str(out), "--pairs", "600", "1200", "2400", "--hidden", "32",
                             "--calls", "2", "--cpu"]) == 0
    data = json.loads(out.read_text())
    assert len(data["rows"]) == 3 and "32" in data["fit_ref"]
    fixed, per = chain_sweep.line_fit([1, 2, 3], [3.0, 5.0, 7.0])
    assert abs(fixed - 1.0) < 1e-9 and abs(per - 2.0) < 1e-9


def test_onesided_verdict_rules():
    from terracemoe_simulator_b200.bench.onesided_vs_collective import verdict
    rows = [{"collective_ms": 0.05, "one_sided_ms": 0.01},      # launch floor: not counted
            {"collective_ms": 0.20, "one_sided_ms": 0.16},
            {"collective_ms": 0.40, "one_sided_ms": 0.30}]
    v = verdict(rows)
    assert v["counted"] == 2 and v["adopt_one_sided"] and 1.25 <= v["median_speedup"] <= 1.34
    assert not verdict(rows, criterion=1.5)["adopt_one_sided"]
    assert verdict(rows[:1])["counted"] == 0 and not verdict([])["adopt_one_sided"]


def test_figures_reproducible_and_wellformed(tmp_path):
    from terracemoe_simulator_b200.tools import gen_figures
    first = gen_figures.generate(str(tmp_path / "a"))
    second = gen_figures.generate(str(tmp_path / "b"))
    assert len(first) == len(gen_figures.FIGURES) >= 18
    for pa, pb in zip(first, second):
        ta, tb = open(pa).read(), open(pb).read()
        assert ta == tb and "nan" not in ta
        xml.dom.minidom.parseString(ta)
    only = gen_figures.generate(str(tmp_path / "c"), only=["f8", "f17"])
    assert [os.path.basename(p) for p in only] == ["f8-breakeven-map.svg", "f17-b200-ratio.svg"]


def test_traffic_helpers():
    import torch
    from terracemoe_simulator_b200.bench import traffic
    from terracemoe_simulator_b200.routing import TRouteConfig
    cfg = TRouteConfig(16, 4, 4, 2)
    group_idx = torch.tensor([[0, 1], [1, 2], [0, 3]])
    src = torch.tensor([0, 2, 5])
    m = traffic.dispatch_traffic(group_idx, src, cfg, cards_per_group=2)
    assert m.shape == (4, 4) and int(m.sum()) == 6
    assert traffic.uniformity_cv(torch.ones(4, 4)) == pytest.approx(0.0)


def test_device_prefetcher_passthrough_and_order():
    import itertools
    import torch
    from terracemoe_simulator_b200.utils.prefetch import DevicePrefetcher
    batches = [torch.full((2, 3), float(i)) for i in range(5)]
    out = list(DevicePrefetcher(batches, "cpu"))
    assert len(out) == 5 and all(torch.equal(a, b) for a, b in zip(out, batches))
    pairs = list(DevicePrefetcher([(torch.ones(1), torch.zeros(2))] * 3, "cpu", depth=1))
    assert len(pairs) == 3 and isinstance(pairs[0], tuple)
    feed = DevicePrefetcher(itertools.cycle(batches), "cpu")
    assert [int(next(feed)[0, 0]) for _ in range(7)] == [0, 1, 2, 3, 4, 0, 1]


def test_device_prefetcher_take_and_refill_keep_the_order():
    """take() hands out the next batch without starting a copy; refill() starts one (on a CPU
    device the ``after`` event is ignored): the order of batches does not change."""
    import itertools
    import torch
    from terracemoe_simulator_b200.utils.prefetch import DevicePrefetcher
    batches = [torch.full((2,), float(i)) for i in range(4)]
    feed = DevicePrefetcher(itertools.cycle(batches), "cpu", depth=2)
    seen = []
    for _ in range(6):
        seen.append(int(feed.take()[0]))
        assert len(feed.queue) == 1
        feed.refill(after=None)
        assert len(feed.queue) == 2
    assert seen == [0, 1, 2, 3, 0, 1]
    short = DevicePrefetcher(batches[:2], "cpu", depth=2)
    short.take(), short.take()
    with pytest.raises(StopIteration):
        short.take()


def test_deferred_scalar_reads_every_value_one_step_late():
    import torch
    from terracemoe_simulator_b200.utils.prefetch import DeferredScalar
    d = DeferredScalar("cpu")
    out = [d.push(torch.tensor(float(i))) for i in range(5)]
    assert out == [None, 0.0, 1.0, 2.0, 3.0] and d.flush() == 4.0 and d.bytes_per_read == 4
    assert DeferredScalar("cpu").flush() is None
    d3 = DeferredScalar("cpu", lag=3)
    out = [d3.push(torch.tensor(float(i))) for i in range(6)]
    assert out == [None, None, None, 0.0, 1.0, 2.0] and d3.flush() == 5.0
    side = DeferredScalar("cpu", lag=2, side_stream=True)        # no stream on a CPU device
    assert side.stream is None
    assert [side.push(torch.tensor(float(i))) for i in range(4)] == [None, None, 0.0, 1.0]


def test_route_results_record_is_consistent():
    from terracemoe_simulator_b200.tools import route_results as rr
    assert abs(rr.conjunction_cost_share() - 0.38) < 0.005           # "38 % of the quota alone"
    for readout in ("20k", "30k"):
        for mode in rr.MODES:
            mean, lo, hi = rr.LOSS_COST[readout][mode]
            assert lo < mean < hi
            seeds = rr.PER_SEED[readout][mode]
            assert len(seeds) == 4 and abs(sum(seeds) / 4 - mean) < 2e-4
    assert all(abs(v[0]) < rr.EQUIVALENCE_PP and -rr.EQUIVALENCE_PP < v[1] and v[2] < rr.EQUIVALENCE_PP
               for v in rr.DOWNSTREAM_PP.values())
    assert abs(sum(rr.STEP_G) / 2 - 0.9976) < 1e-4
    assert max(m[3] for m in rr.FORERUNNER) == dict((m[0], m[3]) for m in rr.FORERUNNER)["full"]


def test_residency_fit_recovers_a_known_profile():
    from terracemoe_simulator_b200.bench import residency as rs
    a, b, c, static, cap = 3.5e4, 2.0e5, 7.0e8, 4.0e10, 180e9
    samples = []
    for L in (4, 8, 16):
        for tok in (4096, 8192):
            peak = static + a * tok * L + b * tok + c
            samples.append(rs.Sample(L, tok, static, peak, peak * 1.05, peak + 9e9))
    prof, d = rs.fit_profile(samples, cap)
    assert prof.measured and abs(prof.activation_bytes_per_token_layer - a) / a < 1e-6
    assert abs(d["per_token"] - b) / b < 1e-6 and d["worst_residual"] < 1e-9
    assert abs(prof.overhead_frac - 9e9 / cap) < 1e-12
    with pytest.raises(ValueError):
        rs.fit_profile(samples[:2], cap)
    with pytest.raises(ValueError):                       # layers never vary
        rs.fit_profile([s for s in samples if s.layers == 4] * 2, cap)
    # a measured profile removes the ASSUMED tag from the memory verdict
    from terracemoe_simulator_b200.sim import codesign
    arch, machine = codesign.REFERENCE_ARCH, codesign.hgx_b200()
    got = codesign.residency(arch, machine, 8, prof)
    assert got["measured"] and got["provenance"]["activation_bytes"].startswith("measured")
    assert codesign.residency(arch, machine, 8)["provenance"]["activation_bytes"].startswith("ASSUMED")


def test_residency_measure_point_with_an_injected_probe():
    from terracemoe_simulator_b200.bench import residency as rs
    calls = []
    probe = (lambda: calls.append("reset"),
             lambda: {"peak_allocated": 5e6, "peak_reserved": 6e6, "device_used": 7e6})
    s = rs.measure_point(2, 1, 16, device="cpu", dim=32, heads=2, experts=4, d_expert=16,
                         d_shared=16, groups=2, top_k=2, top_groups=1, vocab=64, backend="grouped",
                         steps=2, probe=probe)
    assert calls == ["reset"] and s.layers == 2 and s.tokens == 16
    assert s.peak_allocated == 5e6 and s.static_bytes > 0


def test_trace_is_a_noop_unless_enabled_and_accumulates_per_phase(monkeypatch):
    import time
    from terracemoe_simulator_b200.utils import trace
    monkeypatch.delenv("TERRACE_TRACE", raising=False)
    trace.reset()
    assert not trace.enabled()
    assert trace.phase("a") is trace.phase("b")                 # one shared no-op object
    with trace.phase("a"):
        pass
    assert trace.report() == {}
    monkeypatch.setenv("TERRACE_TRACE", "events")
    trace.reset()
    assert trace.enabled()
    for _ in range(3):
        with trace.phase("slow", cuda=False):
            time.sleep(0.01)
        with trace.phase("fast", cuda=False):
            pass
    rep = trace.report()
    assert list(rep) == ["slow", "fast"] and rep["slow"]["calls"] == 3
    assert rep["slow"]["ms"] >= 25.0 > rep["fast"]["ms"]
    assert abs(rep["slow"]["ms_per_call"] - rep["slow"]["ms"] / 3) < 1e-9
    assert "slow" in trace.format_report(rep)
    assert trace.report() == {}                                  # the report reset the totals
    monkeypatch.setenv("TERRACE_TRACE", "0")
    trace.reset()
    assert not trace.enabled()


def test_trace_folds_old_spans_instead_of_growing_without_bound(monkeypatch):
    from terracemoe_simulator_b200.utils import trace
    monkeypatch.setenv("TERRACE_TRACE", "events")
    trace.reset()
    monkeypatch.setattr(trace, "_MAX_PENDING", 8)
    for _ in range(50):
        with trace.phase("p", cuda=False):
            pass
    assert len(trace._SPANS["p"]) <= 8
    assert trace.report()["p"]["calls"] == 50
    monkeypatch.setenv("TERRACE_TRACE", "0")
    trace.reset()


def _check_pdf(blob: bytes):
    """Structural check of a PDF: header, trailer, and every xref offset lands on its object."""
    import re
    assert blob.startswith(b"%PDF-1.4") and blob.rstrip().endswith(b"%%EOF")
    start = int(re.search(rb"startxref\s+(\d+)", blob).group(1))
    assert blob[start:start + 4] == b"xref"
    lines = blob[start:].split(b"\n")
    n = int(lines[1].split()[1])
    for i in range(1, n):
        off = int(lines[2 + i].split()[0])
        assert blob[off:].startswith(b"%d 0 obj" % i), (i, blob[off:off + 12])
    length = int(re.search(rb"/Length (\d+)", blob).group(1))
    body = blob.split(b"stream\n", 1)[1]
    assert body[length:length + 10] == b"\nendstream"
    return body[:length].decode("latin-1")


def test_svg2pdf_converts_every_figure(tmp_path, monkeypatch):
    from terracemoe_simulator_b200.tools import gen_figures, svg2pdf
    from terracemoe_simulator_b200.tools.svgplot import Chart, heatmap
    c = Chart("a (title) with \\ specials", "x", "y")
    c.line([1, 2, 3], [1.0, 4.0, 9.0], label="squares", dash="4,2")
    c.band([1, 2, 3], [0.5, 3.0, 8.0], [1.5, 5.0, 10.0], label="band")
    c.hline(2.0, label="limit")
    stream = _check_pdf(svg2pdf.convert(c.render()))
    assert "(squares) Tj" in stream and "\\(title\\)" in stream and "\\\\ specials" in stream
    assert "/GS1 gs" in stream and "[4 2] 0 d" in stream and " c " in stream     # alpha, dash, circles
    assert "0 -1 -1 0" in stream                                  # the rotated axis label
    _check_pdf(svg2pdf.convert(heatmap([[0.5, 1.5], [1.0, 2.0]], ["a", "b"], ["c", "d"])))
    # anchors use the Helvetica advance widths
    assert abs(svg2pdf.text_width("0123456789", 10.0) - 55.6) < 1e-9
    assert svg2pdf.text_width("iii", 10.0) < svg2pdf.text_width("WWW", 10.0)
    # the switch: off by default, a .pdf beside every .svg when on
    monkeypatch.delenv("TERRACE_FIG_PDF", raising=False)
    assert [os.path.splitext(p)[1] for p in gen_figures.generate(str(tmp_path), ["f8"])] == [".svg"]
    monkeypatch.setenv("TERRACE_FIG_PDF", "1")
    out = gen_figures.generate(str(tmp_path), ["f8", "f14"])
    assert sorted(os.path.splitext(p)[1] for p in out) == [".pdf", ".pdf", ".svg", ".svg"]
    for p in out:
        if p.endswith(".pdf"):
            _check_pdf(open(p, "rb").read())


def _load_root_bench():
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("root_bench", os.path.join(root, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_root_bench_contract_helpers():
    """The parts of the headline benchmark that need no GPU: the configuration both arms report
    (identical keys and values for ours and the reference), block statistics, the clock sampler's
    summary, and the command-line surface."""
    b = _load_root_bench()
    for world in (1, 2, 4, 8):
        cfg = b.bench_config(world)
        assert {"model", "global_batch", "seq_len", "parallelism"} <= set(cfg)
        assert cfg["global_batch"] == b.TOKENS * world and cfg["parallelism"] == "ep%d" % world
        assert cfg["rpn"] == b.RPN[world] and world % cfg["rpn"] == 0
        assert b.ROUTING_GROUPS[world] >= 2
    stats = b.block_stats([70.0, 60.0, 80.0, 65.0, 90.0], steps=20)
    assert stats == {"ms_per_step": 3.5, "ms_min": 3.0, "ms_max": 4.5, "blocks": 5}
    src = open(b.__file__).read()
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--repeats", "--e2e-variant",
                 "--no-ab", "--no-parity"):
        assert flag in src
    assert '"gpu_launches"' in src and '"e2e"' in src and '"clocks"' in src
