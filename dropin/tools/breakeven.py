"""Forwarder: ``python tools/breakeven.py --ratio R`` / ``python -m tools.breakeven``."""
import sys as _sys

try:
    from terracemoe_simulator_b200.tools import breakeven as _impl
except ModuleNotFoundError:     # run as a script from a checkout: the package sits two levels up
    import os as _os
    _sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.dirname(
        _os.path.abspath(__file__)))))
    from terracemoe_simulator_b200.tools import breakeven as _impl

if __name__ == "__main__":
    _rc = _impl.main()
    if _rc:                 # like the reference's script: a clean run returns, it does not exit
        _sys.exit(_rc)
_sys.modules[__name__] = _impl
