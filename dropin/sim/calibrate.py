"""Forwarder to ``terracemoe_simulator_b200.sim.calibrate``; ``python -m sim.calibrate`` runs that module's entry point."""
from terracemoe_simulator_b200.sim.calibrate import *  # noqa: F401,F403
from terracemoe_simulator_b200.sim import calibrate as _impl


def __getattr__(name):
    return getattr(_impl, name)
