"""Forwarder: the reference's ``terrace`` package name on top of ``terracemoe_simulator_b200``."""
from terracemoe_simulator_b200 import *  # noqa: F401,F403
from terracemoe_simulator_b200 import __all__  # noqa: F401
