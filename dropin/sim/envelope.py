"""Forwarder to ``terracemoe_simulator_b200.sim.envelope``; ``python -m sim.envelope`` runs that module's entry point."""
from terracemoe_simulator_b200.sim.envelope import *  # noqa: F401,F403
from terracemoe_simulator_b200.sim import envelope as _impl


def __getattr__(name):
    return getattr(_impl, name)


if __name__ == "__main__":
    import runpy
    runpy.run_module("terracemoe_simulator_b200.sim.envelope", run_name="__main__")
