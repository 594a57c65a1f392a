"""Forwarder to ``terracemoe_simulator_b200.bench.a2a_form_probe``."""
import sys as _sys

from terracemoe_simulator_b200.bench import a2a_form_probe as _impl

if __name__ == "__main__":
    _sys.exit(_impl.main())
_sys.modules[__name__] = _impl
