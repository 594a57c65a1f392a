"""terracemoe_simulator_b200: a Blackwell-native (B200, sm_100a) hierarchical Mixture-of-Experts
expert-parallel framework with T-Route routing, T-A2A two-hop dispatch/combine and an analytic
cost model.

Sub-packages: ``routing`` / ``layer`` (T-Route and MoE layers), ``models`` (TerraceLM decoder,
checkpoints), ``ops`` (native kernels, loader, executable specs), ``parallel`` (one-hop and
two-hop expert parallelism over ``torch.distributed`` and over fused peer-memory kernels),
``sim`` (cost model), ``bench`` (measurement instruments), ``utils`` (drift probe, timing).
"""
from .layer import HierarchicalMoE, SwiGLU, TerracedMoE, grouped_mm
from .routing import Router, TRouteConfig, expert_load, t_route, update_bias_

__all__ = ["TRouteConfig", "t_route", "expert_load", "update_bias_", "Router", "SwiGLU",
           "TerracedMoE", "HierarchicalMoE", "grouped_mm"]
__version__ = "0.1.0"
