"""The reference's ``terrace`` package name: replaced at import by the modules of
``terracemoe_simulator_b200`` (``compat.become`` installs the alias finder and swaps this stub out)."""
from terracemoe_simulator_b200.compat import become

become(__name__)
