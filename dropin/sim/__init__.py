"""Forwarder: the reference's ``sim`` package name on top of ``terracemoe_simulator_b200.sim``."""
from terracemoe_simulator_b200.sim import MODULES  # noqa: F401
from terracemoe_simulator_b200 import sim as _impl


def __getattr__(name):
    return getattr(_impl, name)
