"""Forwarder to ``terracemoe_simulator_b200.parallel.ep``."""
import sys as _sys

import terracemoe_simulator_b200.parallel.ep as _impl

_sys.modules[__name__] = _impl
