from .traffic import dispatch_traffic, traffic_bytes, uniformity_cv

__all__ = ["dispatch_traffic", "traffic_bytes", "uniformity_cv"]
