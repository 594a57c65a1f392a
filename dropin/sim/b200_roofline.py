"""Forwarder to ``terracemoe_simulator_b200.sim.b200_roofline``; ``python -m sim.b200_roofline`` runs that module's entry point."""
from terracemoe_simulator_b200.sim.b200_roofline import *  # noqa: F401,F403
from terracemoe_simulator_b200.sim import b200_roofline as _impl


def __getattr__(name):
    return getattr(_impl, name)


if __name__ == "__main__":
    import runpy
    runpy.run_module("terracemoe_simulator_b200.sim.b200_roofline", run_name="__main__")
