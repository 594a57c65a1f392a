"""Forwarder: traffic helpers of ``terracemoe_simulator_b200.bench``."""
from terracemoe_simulator_b200.bench.traffic import dispatch_traffic, traffic_bytes, uniformity_cv  # noqa: F401
