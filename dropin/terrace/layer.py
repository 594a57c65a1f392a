"""Forwarder to ``terracemoe_simulator_b200.layer``."""
import sys as _sys

import terracemoe_simulator_b200.layer as _impl

_sys.modules[__name__] = _impl
