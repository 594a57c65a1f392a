"""Forwarder: planning helpers of the two-hop dispatch (``terracemoe_simulator_b200.parallel.plan``)."""
import sys as _sys

import terracemoe_simulator_b200.parallel.plan as _impl

_sys.modules[__name__] = _impl
