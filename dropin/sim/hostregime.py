"""Forwarder to ``terracemoe_simulator_b200.sim.hostregime``; ``python -m sim.hostregime`` runs that module's entry point."""
from terracemoe_simulator_b200.sim.hostregime import *  # noqa: F401,F403
from terracemoe_simulator_b200.sim import hostregime as _impl


def __getattr__(name):
    return getattr(_impl, name)


if __name__ == "__main__":
    import runpy
    runpy.run_module("terracemoe_simulator_b200.sim.hostregime", run_name="__main__")
