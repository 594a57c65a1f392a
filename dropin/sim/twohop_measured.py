"""Forwarder to ``terracemoe_simulator_b200.sim.twohop_measured``; ``python -m sim.twohop_measured`` runs that module's entry point."""
from terracemoe_simulator_b200.sim.twohop_measured import *  # noqa: F401,F403
from terracemoe_simulator_b200.sim import twohop_measured as _impl


def __getattr__(name):
    return getattr(_impl, name)


if __name__ == "__main__":
    import runpy
    runpy.run_module("terracemoe_simulator_b200.sim.twohop_measured", run_name="__main__")
