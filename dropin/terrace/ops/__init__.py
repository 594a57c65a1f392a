"""Forwarder to ``terracemoe_simulator_b200.ops``."""
import sys as _sys

import terracemoe_simulator_b200.ops as _impl

_sys.modules[__name__] = _impl
