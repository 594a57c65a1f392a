"""The drop-in forwarders: the reference's import paths and command lines on top of this package."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENV = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.join(ROOT, "dropin"), ROOT]),
           PYTHONIOENCODING="ascii")


def _py(args, cwd="/tmp"):
    return subprocess.run([sys.executable] + args, capture_output=True, env=ENV, cwd=cwd, timeout=600)


def test_reference_import_paths_resolve():
    code = """
from terrace import TRouteConfig, t_route, Router, TerracedMoE
from terrace.layer import grouped_mm, HierarchicalMoE
from terrace.model import ModelArgs, TerraceLM, rmsnorm
from terrace.ep_dist import ep_moe_forward, _a2a, _a2a_raw, _A2A
from terrace.ta2a import plan_ta2a, dispatch_stats
from terrace.ta2a_fwd import init_ta2a_groups, ta2a_moe_forward, build_expansion, fixed_hist
from terrace.ta2a_dispatch import (ta2a_permute, ta2a_unpermute, ta2a_permute_overlap,
                                   ta2a_unpermute_overlap, routing_map_to_topk, ta2a_enabled)
from terrace.ta2a_pack import hopa_pack, hopb_pack_meta, pack_mode, assert_not_aliased
from terrace.ops import k1_arrival, k1_arrival_ref, custom_ops_enabled, status
from terrace.ops.k2_ref import k2_pack_ref
from terrace.drift_probe import note, compare
from sim import ClusterSpec, MoEGeometry, one_hop_call, two_hop_call, HOLDOUTS
from sim.calibrate import flat_supernode
import sim.profile
from bench import dispatch_traffic, uniformity_cv
assert TRouteConfig(16, 4, 4, 2).per_group_k == 2
print(round(sim.profile.byte_breakeven(8, 3), 4))
"""
    proc = _py(["-c", code])
    assert proc.returncode == 0, proc.stderr.decode()[-2000:]
    assert proc.stdout.decode().strip() == "1.3125"


def test_reference_command_lines_run():
    for module in ("sim.sweep", "sim.profile", "sim.validate_micro", "sim.codesign"):
        proc = _py(["-m", module])
        assert proc.returncode == 0, (module, proc.stderr.decode()[-1500:])
        proc.stdout.decode("ascii")
        assert len(proc.stdout) > 100
    proc = _py([os.path.join(ROOT, "dropin", "tools", "breakeven.py"), "--ratio", "9.0"])
    assert proc.returncode == 0 and b"worth an integration experiment" in proc.stdout


def test_pack_errors_are_runtime_errors_too():
    import pytest
    import torch
    from terracemoe_simulator_b200.parallel import pack
    ids = torch.zeros(3, dtype=torch.int64)
    with pytest.raises(RuntimeError):
        pack.hopa_pack(torch.randn(3, 4).bfloat16(), torch.rand(3, 2), ids)
    with pytest.raises(TypeError):
        pack.hopa_pack(torch.randn(3, 4), torch.rand(3, 2), torch.zeros(3, dtype=torch.int32))
    with pytest.raises(RuntimeError):
        pack.hopb_pack_meta(ids, torch.zeros(3, dtype=torch.int64))
    buf = torch.zeros(4, 8, dtype=torch.int64)
    with pytest.raises(RuntimeError, match="shared storage"):
        pack.assert_not_aliased(buf, buf[:, :2])
    pack.assert_not_aliased(buf, buf[:, :2].clone())
