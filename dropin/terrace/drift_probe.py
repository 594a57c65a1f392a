"""Forwarder to ``terracemoe_simulator_b200.utils.drift_probe``."""
import sys as _sys

import terracemoe_simulator_b200.utils.drift_probe as _impl

_sys.modules[__name__] = _impl
