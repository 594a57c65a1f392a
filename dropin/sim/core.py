"""Forwarder to ``terracemoe_simulator_b200.sim.core``; ``python -m sim.core`` runs that module's entry point."""
from terracemoe_simulator_b200.sim.core import *  # noqa: F401,F403
from terracemoe_simulator_b200.sim import core as _impl


def __getattr__(name):
    return getattr(_impl, name)
