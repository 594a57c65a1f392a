"""Forwarder to ``terracemoe_simulator_b200.sim.validate_sweep``; ``python -m sim.validate_sweep`` runs that module's entry point."""
from terracemoe_simulator_b200.sim.validate_sweep import *  # noqa: F401,F403
from terracemoe_simulator_b200.sim import validate_sweep as _impl


def __getattr__(name):
    return getattr(_impl, name)


if __name__ == "__main__":
    import runpy
    runpy.run_module("terracemoe_simulator_b200.sim.validate_sweep", run_name="__main__")
