"""Forwarder to ``terracemoe_simulator_b200.parallel.seams``."""
import sys as _sys

import terracemoe_simulator_b200.parallel.seams as _impl

_sys.modules[__name__] = _impl
