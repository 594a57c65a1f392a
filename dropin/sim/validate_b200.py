"""Forwarder to ``terracemoe_simulator_b200.sim.validate_b200``; ``python -m sim.validate_b200`` runs that module's entry point."""
from terracemoe_simulator_b200.sim.validate_b200 import *  # noqa: F401,F403
from terracemoe_simulator_b200.sim import validate_b200 as _impl


def __getattr__(name):
    return getattr(_impl, name)


if __name__ == "__main__":
    import runpy
    runpy.run_module("terracemoe_simulator_b200.sim.validate_b200", run_name="__main__")
