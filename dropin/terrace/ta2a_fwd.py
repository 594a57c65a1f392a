"""Forwarder: closed two-hop forward and its wire helpers (``terracemoe_simulator_b200.parallel.ta2a``)."""
from terracemoe_simulator_b200.compat import _expand_arrival_quota, _pack_quota_wire  # noqa: F401
from terracemoe_simulator_b200.ops.refs import fixed_hist, stable_bucket_order  # noqa: F401
from terracemoe_simulator_b200.ops.refs import stable_bucket_order as _stable_argsort_small  # noqa: F401
from terracemoe_simulator_b200.parallel.ta2a import (build_expansion, get_ta2a_groups,  # noqa: F401
                                                     init_ta2a_groups, ta2a_moe_forward)
