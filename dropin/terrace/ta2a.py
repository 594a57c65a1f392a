"""Forwarder: planning helpers of the two-hop dispatch (``terracemoe_simulator_b200.parallel.plan``)."""
from terracemoe_simulator_b200.parallel.plan import dispatch_stats, plan_ta2a, reset_plan_cache  # noqa: F401
