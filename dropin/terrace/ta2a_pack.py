"""Forwarder to ``terracemoe_simulator_b200.parallel.pack``."""
import sys as _sys

import terracemoe_simulator_b200.parallel.pack as _impl

_sys.modules[__name__] = _impl
