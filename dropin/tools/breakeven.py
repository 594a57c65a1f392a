"""Forwarder: ``python tools/breakeven.py --ratio R`` / ``python -m tools.breakeven``."""
import sys as _sys

from terracemoe_simulator_b200.tools import breakeven as _impl

if __name__ == "__main__":
    _sys.exit(_impl.main())
_sys.modules[__name__] = _impl
