"""Forwarder: closed two-hop forward and its wire helpers (``terracemoe_simulator_b200.parallel.ta2a``)."""
from terracemoe_simulator_b200.ops.refs import fixed_hist, stable_bucket_order  # noqa: F401
from terracemoe_simulator_b200.parallel.ta2a import (build_expansion, get_ta2a_groups, init_ta2a_groups,  # noqa: F401
                                  ta2a_moe_forward)
