"""Drop-in module aliases: make ``import terrace`` / ``import sim`` resolve to this package.

``install_aliases()`` registers the reference's module names in ``sys.modules``:
``terrace`` (routing, layer, model, ep_dist, ta2a, ta2a_fwd, ta2a_dispatch, ta2a_pack,
drift_probe, ops, ops.k2_ref), ``sim`` and its sub-modules, and ``bench``.  Names the reference
exposes under different module boundaries (``ta2a`` = plan, ``ta2a_fwd`` = closed forward +
wire helpers) are re-exported by small namespace modules.
"""
from __future__ import annotations

import importlib
import sys
import types

_PKG = "terracemoe_simulator_b200"


def _module(name: str, **attrs) -> types.ModuleType:
    mod = types.ModuleType(name)
    mod.__dict__.update(attrs)
    sys.modules[name] = mod
    return mod


# ---- adapters with the reference's private helper signatures (its tests import them) ----------
def _expand_arrival_quota(rslot):
    """Quota slot table ``[R, q]`` -> row-major ``(r_idx, slot_idx)`` pairs
    (``terrace/ta2a_fwd.py:252-266`` in the reference)."""
    import torch
    R, quota = rslot.shape
    r_idx = torch.arange(R, device=rslot.device, dtype=torch.int64).unsqueeze(1).expand(
        R, quota).reshape(-1)
    return r_idx, rslot.reshape(-1)


def _pack_quota_wire(expert_idx, gates, inverse, payload, n_rows: int, slots: int, quota: int,
                     n_experts: int, *, sorted_rows: bool = False):
    """Quota wire planes with the reference's argument list (``terrace/ta2a_fwd.py:177-249``):
    returns ``(slot_table[n_rows, quota] ascending, gate_table[n_rows, quota])``."""
    import torch
    from .parallel.ta2a import pack_quota_wire
    T, k = expert_idx.shape
    if payload is not None and gates.dtype != payload.dtype:
        raise RuntimeError(f"gate dtype {gates.dtype} != payload dtype {payload.dtype}: the gate "
                           f"plane travels in the payload dtype; cast at the caller")
    inv = inverse.view(T, k)
    if not sorted_rows:
        order = torch.argsort(expert_idx, dim=1, stable=True)
        expert_idx, gates, inv = (expert_idx.gather(1, order), gates.gather(1, order),
                                  inv.gather(1, order))
    slot_tab, gate_tab, _rows = pack_quota_wire(expert_idx, gates, inv.reshape(-1), n_rows, slots,
                                                quota)
    return slot_tab, gate_tab


def install_aliases(force: bool = False) -> None:
    if "terrace" in sys.modules and not force:
        return
    imp = importlib.import_module
    routing, layer = imp(f"{_PKG}.routing"), imp(f"{_PKG}.layer")
    model = imp(f"{_PKG}.models.decoder")
    ep, plan = imp(f"{_PKG}.parallel.ep"), imp(f"{_PKG}.parallel.plan")
    ta2a, seams = imp(f"{_PKG}.parallel.ta2a"), imp(f"{_PKG}.parallel.seams")
    pack, probe = imp(f"{_PKG}.parallel.pack"), imp(f"{_PKG}.utils.drift_probe")
    ops, refs = imp(f"{_PKG}.ops"), imp(f"{_PKG}.ops.refs")
    top = imp(_PKG)
    terrace = _module("terrace", **{k: getattr(top, k) for k in top.__all__})
    terrace.__path__ = []
    pairs = {"routing": routing, "layer": layer, "model": model, "ep_dist": ep,
             "ta2a_dispatch": seams, "ta2a_pack": pack, "drift_probe": probe, "ops": ops}
    for name, mod in pairs.items():
        sys.modules[f"terrace.{name}"] = mod
        setattr(terrace, name, mod)
    sys.modules["terrace.ta2a"] = plan
    fwd = {k: getattr(ta2a, k) for k in ("init_ta2a_groups", "ta2a_moe_forward",
                                         "build_expansion", "fixed_hist")}
    fwd["_stable_argsort_small"] = refs.stable_bucket_order
    fwd["_expand_arrival_quota"] = _expand_arrival_quota
    fwd["_pack_quota_wire"] = _pack_quota_wire
    sys.modules["terrace.ta2a_fwd"] = _module("terrace.ta2a_fwd", **fwd)
    sys.modules["terrace.ops.k2_ref"] = _module("terrace.ops.k2_ref", k2_pack_ref=refs.k2_pack_ref)
    sim = imp(f"{_PKG}.sim")
    sys.modules["sim"] = sim
    for name in sim.MODULES:
        sys.modules[f"sim.{name}"] = imp(f"{_PKG}.sim.{name}")
    sys.modules["bench"] = imp(f"{_PKG}.bench")
