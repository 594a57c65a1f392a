"""Forwarder to ``terracemoe_simulator_b200.bench.twohop_verdict``."""
import sys as _sys

from terracemoe_simulator_b200.bench import twohop_verdict as _impl

if __name__ == "__main__":
    _sys.exit(_impl.main())
_sys.modules[__name__] = _impl
