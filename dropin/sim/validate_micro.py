"""Forwarder to ``terracemoe_simulator_b200.sim.validate_micro``; ``python -m sim.validate_micro`` runs that module's entry point."""
from terracemoe_simulator_b200.sim.validate_micro import *  # noqa: F401,F403
from terracemoe_simulator_b200.sim import validate_micro as _impl


def __getattr__(name):
    return getattr(_impl, name)


if __name__ == "__main__":
    import runpy
    runpy.run_module("terracemoe_simulator_b200.sim.validate_micro", run_name="__main__")
