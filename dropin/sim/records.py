"""Forwarder to ``terracemoe_simulator_b200.sim.records``; ``python -m sim.records`` runs that module's entry point."""
from terracemoe_simulator_b200.sim.records import *  # noqa: F401,F403
from terracemoe_simulator_b200.sim import records as _impl


def __getattr__(name):
    return getattr(_impl, name)
