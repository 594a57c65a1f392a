"""Forwarder to ``terracemoe_simulator_b200.sim.hierarchy``; ``python -m sim.hierarchy`` runs that module's entry point."""
from terracemoe_simulator_b200.sim.hierarchy import *  # noqa: F401,F403
from terracemoe_simulator_b200.sim import hierarchy as _impl


def __getattr__(name):
    return getattr(_impl, name)


if __name__ == "__main__":
    import runpy
    runpy.run_module("terracemoe_simulator_b200.sim.hierarchy", run_name="__main__")
