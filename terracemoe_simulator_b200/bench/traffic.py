"""Group-level traffic matrix of a routing decision.

``dispatch_traffic`` counts, per (source group, destination group), the messages a T-A2A
dispatch sends (one per distinct (token, destination group)); ``traffic_bytes`` scales by the row
size; ``uniformity_cv`` is the coefficient of variation of the off-diagonal entries.  Counterpart
of the reference's ``bench/traffic.py`` (:15-36).
"""
from __future__ import annotations

import torch


def dispatch_traffic(group_idx: torch.Tensor, src_card: torch.Tensor, cfg,
                     cards_per_group: int) -> torch.Tensor:
    """``group_idx[T, M]`` destination groups per token, ``src_card[T]`` the card holding each
    token -> ``[N_g, N_g]`` message counts as float32 (token-level dedup: one per (token, group))."""
    n = cfg.n_groups
    src_group = torch.div(src_card, cards_per_group, rounding_mode="floor").long()
    T, M = group_idx.shape
    flat = (src_group.unsqueeze(1).expand(T, M) * n + group_idx.long()).reshape(-1)
    out = torch.zeros(n * n, dtype=torch.float32, device=group_idx.device)
    out.scatter_add_(0, flat, torch.ones_like(flat, dtype=torch.float32))
    return out.view(n, n)


def traffic_bytes(matrix: torch.Tensor, hidden: int, bytes_per_elem: int = 2) -> torch.Tensor:
    return matrix * hidden * bytes_per_elem


def uniformity_cv(matrix: torch.Tensor) -> float:
    n = matrix.shape[0]
    off = matrix[~torch.eye(n, dtype=torch.bool, device=matrix.device)].float()
    if off.numel() == 0 or float(off.mean()) == 0.0:
        return 0.0
    return float(off.std(unbiased=False) / off.mean())
