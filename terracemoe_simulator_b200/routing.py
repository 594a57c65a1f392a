"""T-Route: group-limited, equal-quota top-k gating.

Per token the router picks ``top_groups`` (M) expert groups out of ``n_groups`` (N_g) and then
``top_k / top_groups`` (q) experts inside every picked group, so a token's experts always
span exactly M groups with exactly q experts in each.  Selection scores are the sigmoid
affinities plus a per-expert balancing bias; the gate values that weight the expert outputs
come from the *raw* affinities, renormalised over the k picks.

Behavioural parity with the reference ``terrace/routing.py``:
  * ``TRouteConfig`` validation            -> routing.py:20-42
  * ``t_route`` and its four modes         -> routing.py:45-96
  * ``expert_load`` / ``update_bias_``     -> routing.py:112-121
  * ``Router`` (weight init, bias buffer)  -> routing.py:124-134

On a B200 with the native ops enabled, ``Router.forward`` in mode ``"full"`` runs the fused
select kernel (sigmoid, bias, group scores, top-M groups, per-group top-q, gate renormalise,
expert histogram in one launch); the PyTorch code below is the oracle it is tested against.
An optional softmax scoring function is provided for architectures that gate with softmax.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

ROUTING_MODES = ("full", "group_limited", "quota_only", "global_topk")
SCORE_FUNCS = ("sigmoid", "softmax")


@dataclass(frozen=True)
class TRouteConfig:
    """Static routing geometry: E experts in N_g equal groups, k picks over M groups."""

    n_experts: int
    n_groups: int
    top_k: int
    top_groups: int
    group_score_pool: int = 2

    def __post_init__(self):
        if self.n_experts <= 0 or self.n_groups <= 0 or self.top_k <= 0 or self.top_groups <= 0:
            raise ValueError("routing geometry must be positive")
        if self.n_experts % self.n_groups != 0:
            raise ValueError(
                f"n_experts={self.n_experts} must divide evenly into n_groups={self.n_groups}")
        if self.top_k % self.top_groups != 0:
            raise ValueError(
                f"top_k={self.top_k} must divide evenly into top_groups={self.top_groups}")
        if self.top_groups > self.n_groups:
            raise ValueError("top_groups cannot exceed n_groups")
        if self.per_group_k > self.group_size:
            raise ValueError(
                f"per-group quota {self.per_group_k} exceeds group size {self.group_size}")

    @property
    def group_size(self) -> int:
        return self.n_experts // self.n_groups

    @property
    def per_group_k(self) -> int:
        return self.top_k // self.top_groups


def _group_scores(sg: torch.Tensor, pool: int) -> torch.Tensor:
    """Score of a group = mean of its ``pool`` best selection scores. sg: [T, N_g, g]."""
    width = min(pool, sg.shape[-1])
    return sg.topk(width, dim=-1).values.mean(dim=-1)


def t_route(affinity: torch.Tensor, bias: torch.Tensor, cfg: TRouteConfig, mode: str = "full"):
    """Route ``affinity[T, E]`` -> ``(expert_idx[T, k] int64, gates[T, k], group_idx)``.

    ``group_idx`` is ``[T, M]`` for the group-limited modes, ``[T, N_g]`` for ``quota_only``
    and ``[T, k]`` (group of every pick) for ``global_topk``.  Column order of
    ``expert_idx`` in mode ``full``: groups by descending group score, inside a group by
    descending biased affinity.  A mode outside :data:`ROUTING_MODES` raises ``ValueError``.
    """
    if mode not in ROUTING_MODES:
        raise ValueError(f"unknown routing mode {mode!r}; expected one of {ROUTING_MODES}")
    if affinity.dim() != 2 or affinity.shape[1] != cfg.n_experts:
        raise ValueError(f"affinity must be [T, {cfg.n_experts}], got {tuple(affinity.shape)}")
    T = affinity.shape[0]
    g, ng, k, m, q = cfg.group_size, cfg.n_groups, cfg.top_k, cfg.top_groups, cfg.per_group_k
    select = affinity + bias
    by_group = select.view(T, ng, g)
    dev = affinity.device

    if mode == "global_topk":
        expert_idx = select.topk(k, dim=-1).indices
        group_idx = expert_idx // g
    elif mode == "quota_only":
        if k % ng != 0 or k // ng < 1:
            raise ValueError(
                f"quota_only needs top_k ({k}) to be a positive multiple of n_groups ({ng})")
        local = by_group.topk(k // ng, dim=-1).indices                    # [T, N_g, k/N_g]
        offs = (torch.arange(ng, device=dev) * g).view(1, ng, 1)
        expert_idx = (offs + local).reshape(T, -1)
        group_idx = torch.arange(ng, device=dev).expand(T, ng)
    else:
        group_idx = _group_scores(by_group, cfg.group_score_pool).topk(m, dim=-1).indices
        cand = by_group.gather(1, group_idx.unsqueeze(-1).expand(T, m, g))  # [T, M, g]
        if mode == "full":
            local = cand.topk(q, dim=-1).indices                          # [T, M, q]
            expert_idx = (group_idx.unsqueeze(-1) * g + local).reshape(T, k)
        else:  # group_limited: free top-k over the M*g candidates, no quota
            flat = cand.reshape(T, m * g).topk(k, dim=-1).indices         # [T, k] in [0, M*g)
            which = flat // g
            expert_idx = group_idx.gather(1, which) * g + flat % g

    gates = affinity.gather(1, expert_idx)
    gates = gates / gates.sum(dim=-1, keepdim=True)
    return expert_idx, gates, group_idx


def expert_load(expert_idx: torch.Tensor, n_experts: int) -> torch.Tensor:
    """Float histogram of picks per expert (length ``n_experts``); no host sync."""
    flat = expert_idx.reshape(-1)
    out = torch.zeros(n_experts, dtype=torch.float32, device=flat.device)
    return out.scatter_add_(0, flat, torch.ones_like(flat, dtype=torch.float32))


@torch.no_grad()
def update_bias_(bias: torch.Tensor, load: torch.Tensor, gamma: float) -> torch.Tensor:
    """Aux-loss-free balancing: ``bias += gamma * sign(mean(load) - load)`` in place."""
    bias.add_(torch.sign(load.mean() - load).to(bias.dtype), alpha=gamma)
    return bias


def score_affinity(logits: torch.Tensor, score_func: str = "sigmoid") -> torch.Tensor:
    if score_func == "sigmoid":
        return torch.sigmoid(logits)
    if score_func == "softmax":
        return torch.softmax(logits.float(), dim=-1).to(logits.dtype)
    raise ValueError(f"unknown score_func {score_func!r}; expected one of {SCORE_FUNCS}")


class Router(torch.nn.Module):
    """Linear router ``weight[E, hidden]`` + persistent selection ``bias[E]`` buffer."""

    def __init__(self, hidden_size: int, cfg: TRouteConfig, score_func: str = "sigmoid"):
        super().__init__()
        if score_func not in SCORE_FUNCS:
            raise ValueError(f"unknown score_func {score_func!r}; expected one of {SCORE_FUNCS}")
        self.cfg = cfg
        self.score_func = score_func
        self.weight = torch.nn.Parameter(torch.empty(cfg.n_experts, hidden_size))
        torch.nn.init.normal_(self.weight, std=hidden_size ** -0.5)
        self.register_buffer("bias", torch.zeros(cfg.n_experts))

    def forward(self, hidden: torch.Tensor, mode: str = "full"):
        if mode not in ROUTING_MODES:
            raise ValueError(f"unknown routing mode {mode!r}; expected one of {ROUTING_MODES}")
        from . import ops  # deferred: ops imports nothing from routing, but keep import light
        if (mode == "full" and self.score_func == "sigmoid" and hidden.is_cuda
                and ops.custom_ops_enabled() and ops.router_supported(self.cfg, hidden)):
            return ops.fused_route(hidden, self.weight, self.bias, self.cfg)
        affinity = score_affinity(hidden @ self.weight.t().to(hidden.dtype), self.score_func)
        return t_route(affinity.float() if affinity.dtype != torch.float32 else affinity,
                       self.bias.float(), self.cfg, mode)
