"""Analytic cost model of one-hop against two-hop expert-parallel dispatch.

Every module is runnable as ``python -m terracemoe_simulator_b200.sim.<name>``.  The package
exports its main names lazily (``ClusterSpec``, ``MoEGeometry``, ``one_hop_call``,
``two_hop_call``, ``step_delta``, ``HOLDOUTS``, ``validate``) so that running a sub-module with
``-m`` does not import it twice.  Counterpart of the reference's ``sim/__init__.py`` (:48-64).
"""
from __future__ import annotations

import importlib

MODULES = ("core", "calibrate", "fit", "validate_micro", "validate_sweep", "validate", "sweep",
           "uncertainty", "profile", "platforms", "compute", "imbalance", "machine", "codesign",
           "envelope", "archsearch", "overlap", "phase", "record", "hostregime", "hierarchy",
           "tiers", "twohop_measured", "chain_remeasured", "records", "validate_b200", "b200_step",
           "b200_roofline")

_LAZY = {"ClusterSpec": "core", "MoEGeometry": "core", "Level": "core", "one_hop_call": "core",
         "two_hop_call": "core", "step_delta": "core", "HOLDOUTS": "validate",
         "validate": "validate"}

__all__ = sorted(_LAZY)


def __getattr__(name: str):
    if name in _LAZY:
        return getattr(importlib.import_module(f"{__name__}.{_LAZY[name]}"), name)
    if name in MODULES:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
