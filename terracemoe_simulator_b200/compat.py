"""Drop-in module aliases: make ``import terrace`` / ``import sim`` resolve to this package.

``install_aliases()`` registers the reference's ``terrace`` names in ``sys.modules`` (routing,
layer, model, ep_dist, ta2a, ta2a_fwd, ta2a_dispatch, ta2a_pack, drift_probe, ops, ops.k2_ref;
names the reference exposes under different module boundaries -- ``ta2a`` = plan, ``ta2a_fwd`` =
closed forward + wire helpers -- are re-exported by small namespace modules) and puts an
``AliasFinder`` on ``sys.meta_path`` that resolves ``sim``, ``sim.<module>``, ``bench`` and
``tools`` to the modules of this package.  The finder hands out the real module objects (one copy
of every module's state) and its loader answers ``get_code`` under the alias, which is what
``python -m sim.profile`` needs.  The four packages under ``dropin/`` call ``become()`` so that
putting that folder on ``PYTHONPATH`` is enough.
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.machinery
import importlib.util
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


ALIASED_PACKAGES = {"sim": f"{_PKG}.sim", "bench": f"{_PKG}.bench", "tools": f"{_PKG}.tools"}


class _AliasLoader(importlib.abc.Loader):
    """Loads nothing: hands out the real module, and its code when asked under the alias."""

    def __init__(self, real: str):
        self.real = real

    def _module(self):
        return importlib.import_module(self.real)

    def create_module(self, spec):
        # the import system stamps the alias spec on the module it gets back; that is wanted:
        # ``runpy`` looks a loaded module's spec up in ``sys.modules`` and asks ITS loader for the
        # code under the alias name, which only this loader answers
        return self._module()

    def exec_module(self, module) -> None:
        return None

    def get_code(self, fullname):
        return self._module().__loader__.get_code(self.real)

    def get_source(self, fullname):
        return self._module().__loader__.get_source(self.real)

    def is_package(self, fullname) -> bool:
        return hasattr(self._module(), "__path__")


class AliasFinder(importlib.abc.MetaPathFinder):
    """``sim`` / ``bench`` / ``tools`` and their sub-modules -> the modules of this package."""

    def find_spec(self, fullname, path=None, target=None):
        head, _, tail = fullname.partition(".")
        base = ALIASED_PACKAGES.get(head)
        if base is None:
            return None
        real = base + ("." + tail if tail else "")
        try:
            module = importlib.import_module(real)
        except ModuleNotFoundError as exc:
            if exc.name == real:
                return None
            raise
        return importlib.machinery.ModuleSpec(fullname, _AliasLoader(real),
                                              origin=getattr(module, "__file__", None),
                                              is_package=hasattr(module, "__path__"))


def _install_finder() -> None:
    if not any(isinstance(f, AliasFinder) for f in sys.meta_path):
        sys.meta_path.insert(0, AliasFinder())


def become(alias: str) -> None:
    """Called by ``dropin/<alias>/__init__.py``: replace that stub package by the real one."""
    install_aliases()
    if alias in ALIASED_PACKAGES:
        sys.modules[alias] = importlib.import_module(ALIASED_PACKAGES[alias])


def install_aliases(force: bool = False) -> None:
    _install_finder()
    if isinstance(sys.modules.get("terrace"), types.ModuleType) and \
            getattr(sys.modules["terrace"], "_terrace_alias", False) and not force:
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
    terrace.__all__ = list(top.__all__)
    terrace._terrace_alias = True
    pairs = {"routing": routing, "layer": layer, "model": model, "ep_dist": ep,
             "ta2a_dispatch": seams, "ta2a_pack": pack, "drift_probe": probe, "ops": ops}
    for name, mod in pairs.items():
        sys.modules[f"terrace.{name}"] = mod
        setattr(terrace, name, mod)
    sys.modules["terrace.ta2a"] = plan
    fwd = {k: getattr(ta2a, k) for k in ("init_ta2a_groups", "get_ta2a_groups",
                                         "ta2a_moe_forward", "build_expansion", "fixed_hist")}
    fwd["_stable_argsort_small"] = refs.stable_bucket_order
    fwd["_expand_arrival_quota"] = _expand_arrival_quota
    fwd["_pack_quota_wire"] = _pack_quota_wire
    sys.modules["terrace.ta2a_fwd"] = _module("terrace.ta2a_fwd", **fwd)
    sys.modules["terrace.ops.k2_ref"] = _module("terrace.ops.k2_ref", k2_pack_ref=refs.k2_pack_ref)
    for alias, real in ALIASED_PACKAGES.items():        # sub-modules resolve through the finder
        stub = sys.modules.get(alias)
        if stub is None or getattr(stub, "__name__", alias) == alias:
            sys.modules[alias] = imp(real)
