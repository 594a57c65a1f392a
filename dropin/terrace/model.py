"""Forwarder to ``terracemoe_simulator_b200.models.decoder``."""
import sys as _sys

import terracemoe_simulator_b200.models.decoder as _impl

_sys.modules[__name__] = _impl
