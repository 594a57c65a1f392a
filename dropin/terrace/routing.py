"""Forwarder to ``terracemoe_simulator_b200.routing``."""
import sys as _sys

import terracemoe_simulator_b200.routing as _impl

_sys.modules[__name__] = _impl
