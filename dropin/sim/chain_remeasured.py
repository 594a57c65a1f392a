"""Forwarder to ``terracemoe_simulator_b200.sim.chain_remeasured``; ``python -m sim.chain_remeasured`` runs that module's entry point."""
from terracemoe_simulator_b200.sim.chain_remeasured import *  # noqa: F401,F403
from terracemoe_simulator_b200.sim import chain_remeasured as _impl


def __getattr__(name):
    return getattr(_impl, name)


if __name__ == "__main__":
    import runpy
    runpy.run_module("terracemoe_simulator_b200.sim.chain_remeasured", run_name="__main__")
