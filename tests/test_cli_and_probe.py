"""Every cost-model entry point and the breakeven CLI run and print plain ASCII; drift probe."""
import os
import subprocess
import sys

import pytest
import torch

from terracemoe_simulator_b200.sim import MODULES
from terracemoe_simulator_b200.utils import drift_probe as dp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUNNABLE = [m for m in MODULES if m not in ("core", "calibrate", "records")]


def _run(args):
    env = dict(os.environ, PYTHONIOENCODING="ascii", PYTHONPATH=ROOT)
    return subprocess.run([sys.executable] + args, capture_output=True, env=env, cwd=ROOT,
                          timeout=600)


@pytest.mark.parametrize("module", RUNNABLE)
def test_sim_entry_points_print_ascii(module):
    if module in ("fit", "hostregime"):
        pytest.importorskip("scipy")
    proc = _run(["-m", f"terracemoe_simulator_b200.sim.{module}"])
    assert proc.returncode == 0, proc.stderr.decode(errors="replace")[-2000:]
    proc.stdout.decode("ascii")                     # raises on any non-ASCII byte
    assert len(proc.stdout) > 40


@pytest.mark.parametrize("ratio,phrase", [("0.8", "too flat"), ("1.03", "marginal case"),
                                          ("9.0", "worth an integration experiment")])
def test_breakeven_cli_reaches_all_three_verdicts(ratio, phrase):
    proc = _run(["-m", "terracemoe_simulator_b200.tools.breakeven", "--ratio", ratio])
    out = proc.stdout.decode("ascii")
    assert proc.returncode == 0 and phrase in out
    proc2 = _run(["-m", "terracemoe_simulator_b200.tools.breakeven", "--dedup", "--dies", "2"])
    assert b"die-level dedup" in proc2.stdout and b"--ratio" in proc2.stdout


def test_compat_aliases():
    from terracemoe_simulator_b200 import compat
    compat.install_aliases(force=True)
    import sim                                     # noqa: F401  (alias of the cost model)
    import terrace
    from terrace.ta2a import plan_ta2a             # noqa: F401
    from terrace.ta2a_fwd import ta2a_moe_forward  # noqa: F401
    from terrace.ops.k2_ref import k2_pack_ref     # noqa: F401
    assert terrace.TRouteConfig(8, 2, 2, 1).group_size == 4
    assert sim.ClusterSpec.__name__ == "ClusterSpec"
    for name in ("terrace", "sim", "bench"):
        for key in [k for k in sys.modules if k == name or k.startswith(name + ".")]:
            sys.modules.pop(key)


def test_drift_probe_notes_contracts_and_compare(monkeypatch, tmp_path):
    lines = []
    dp.reset()
    dp.set_sink(lines.append)
    try:
        dp.note("off.point", torch.ones(3))
        assert lines == []                          # default: off
        monkeypatch.setenv("TERRACE_DRIFT_PROBE", "1")
        dp.reset()
        dp.set_where(step=3, layer=7)
        dp.tick_dispatch()
        x = torch.arange(12.0).view(3, 4)
        dp.note("seam.rx", x)
        dp.note("seam.rx.perm", x[torch.tensor([2, 0, 1])])       # permutation invariant
        dp.note_int("seam.slot", torch.tensor([3, 1, 2]))
        dp.note_layout("seam.layout", x.t())
        assert lines[0].startswith(dp.PREFIX) and "pt=seam.rx" in lines[0] and "step=3" in lines[0]
        a, b = dp.parse_line(lines[0]), dp.parse_line(lines[1])
        assert a["sabs"] == b["sabs"] and a["ssq"] == b["ssq"] and a["n"] == "12"
        assert "isum=6" in lines[2] and "contig=0" in lines[3]
        assert dp.check_equal("c.same", x, x.clone())
        assert not dp.check_equal("c.diff", x, x + 1)
        assert any("MISMATCH" in l for l in lines)
        idx = torch.tensor([0, 1, 0, 2])
        src = torch.randn(4, 5)
        out = torch.zeros(3, 5).index_add_(0, idx, src)
        assert dp.check_reduction("c.red", out, src, idx, 3)
        monkeypatch.setenv("TERRACE_DRIFT_PROBE_STRICT", "1")
        dp.reset()
        dp.set_sink(lines.append)
        with pytest.raises(dp.DriftProbeMismatch):
            dp.check_equal("c.strict", x, x + 1)
        monkeypatch.delenv("TERRACE_DRIFT_PROBE_STRICT")
        dp.reset()
        dp.set_sink(lines.append)
        dp.note("bad", object())                    # probe error: disables itself, never raises
        assert not dp.enabled()
    finally:
        dp.set_sink(None)
        dp.reset()
    log_a, log_b = tmp_path / "a.log", tmp_path / "b.log"
    rec = "[terrace-drift] pt=%s step=1 layer=0 call=1 rank=0 dt=float32 n=4 sabs=%s ssq=2.0 amax=1.0\n"
    log_a.write_text(rec % ("p1", "1.0") + rec % ("p2", "5.0"))
    log_b.write_text(rec % ("p1", "1.0") + rec % ("p2", "5.5"))
    problems = dp.compare(str(log_a), str(log_b))
    assert len(problems) == 1 and problems[0].startswith("FIRST-DIVERGENCE pt=p2")
    assert dp.main(["compare", str(log_a), str(log_a)]) == 0
    assert dp.main(["compare", str(log_a), str(log_b)]) == 1


def test_environment_switches_are_strict(monkeypatch):
    """Unknown values raise; unset means the documented default."""
    from terracemoe_simulator_b200.utils import flags, trace
    monkeypatch.delenv("TERRACE_EP_OVERLAP", raising=False)
    assert flags.flag_bool("TERRACE_EP_OVERLAP") is False
    assert flags.flag_bool("TERRACE_EP_OVERLAP", True) is True       # the transport's default
    for v, want in (("1", True), ("on", True), ("0", False), ("", False), ("No", False)):
        monkeypatch.setenv("TERRACE_EP_OVERLAP", v)
        assert flags.flag_bool("TERRACE_EP_OVERLAP") is want
    monkeypatch.setenv("TERRACE_EP_OVERLAP", "maybe")
    with pytest.raises(ValueError):
        flags.flag_bool("TERRACE_EP_OVERLAP")
    monkeypatch.setenv("TERRACE_ATTENTION", "flash")
    with pytest.raises(ValueError):
        flags.flag_choice("TERRACE_ATTENTION", ("native", "sdpa"), "native")
    monkeypatch.setenv("TERRACE_EP_PIPELINE", "two")
    with pytest.raises(ValueError):
        flags.flag_int("TERRACE_EP_PIPELINE", 1, 1, 8)
    monkeypatch.setenv("TERRACE_EP_PIPELINE", "3")
    assert flags.flag_int("TERRACE_EP_PIPELINE", 1, 1, 8) == 3
    monkeypatch.setenv("TERRACE_GEMM_PAIR", "sometimes")
    with pytest.raises(ValueError):
        flags.check_native_flags()
    monkeypatch.setenv("TERRACE_GEMM_PAIR", "auto")
    flags.check_native_flags()
    monkeypatch.setenv("TERRACE_TRACE", "everything")
    trace.reset()
    with pytest.raises(ValueError):
        trace.enabled()
    monkeypatch.setenv("TERRACE_TRACE", "0")
    trace.reset()
    assert not trace.enabled()
