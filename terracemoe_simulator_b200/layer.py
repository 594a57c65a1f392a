"""Terraced-MoE layers (single device): SwiGLU, block-diagonal grouped matmul, TerracedMoE,
HierarchicalMoE.

Parity with the reference ``terrace/layer.py``:
  * ``SwiGLU``            -> layer.py:19-27   (``w13`` packs gate|up halves as ``chunk(2, -1)``)
  * ``grouped_mm``        -> layer.py:30-74   (rows pre-sorted by expert, explicit backward)
  * ``TerracedMoE``       -> layer.py:77-130  (``loop`` / ``grouped`` backends, shared expert,
                                              stats dict, in-forward bias update when training)
  * ``HierarchicalMoE``   -> layer.py:133-188 (tier-0 all tokens, tier-1 hardest fraction p)

New relative to the reference: ``expert_backend="native"`` runs the routed experts through the
sm_100a kernels (fused permute, tcgen05 grouped SwiGLU GEMMs, deterministic gate-weighted
combine); ``capacity_factor`` bounds the rows an expert accepts (see ``apply_capacity``).  The
expert-parallel layer lives in ``parallel/moe_layer.py``.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .routing import Router, TRouteConfig, expert_load, t_route, update_bias_

EXPERT_BACKENDS = ("loop", "grouped", "native")


class SwiGLU(nn.Module):
    """``inter = 0`` is allowed and contributes zero: the module then still owns its two
    (zero-element) weights, so that a layer without a shared expert carries the same state-dict
    keys as the reference's (``terrace/layer.py:88`` always builds the shared SwiGLU)."""

    def __init__(self, hidden: int, inter: int):
        super().__init__()
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # "initializing zero-element tensors is a no-op"
            self.w13 = nn.Linear(hidden, 2 * inter, bias=False)
            self.w2 = nn.Linear(inter, hidden, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.w2.in_features == 0:
            return torch.zeros_like(x)
        from . import ops
        if x.is_cuda and ops.custom_ops_enabled() and ops.dense_supported(x, self.w13.weight):
            return ops.swiglu_ffn(x, self.w13.weight, self.w2.weight)
        gate, up = self.w13(x).chunk(2, dim=-1)
        return self.w2(F.silu(gate) * up)


def _segments(counts) -> list[tuple[int, int, int]]:
    """(group, start, stop) for every non-empty group; one host read of ``counts``."""
    sizes = counts.tolist() if torch.is_tensor(counts) else list(counts)
    out, start = [], 0
    for g, n in enumerate(sizes):
        n = int(n)
        if n:
            out.append((g, start, start + n))
        start += n
    return out


def _grouped_mm_plain(x: torch.Tensor, w: torch.Tensor, counts) -> torch.Tensor:
    """x[N, in] (rows sorted by group) times w[E, in, out] block-diagonally -> [N, out]."""
    out = x.new_empty(x.shape[0], w.shape[-1])
    stop = 0
    for g, start, stop in _segments(counts):
        torch.matmul(x[start:stop], w[g], out=out[start:stop])
    if stop < x.shape[0]:
        out[stop:].zero_()          # rows past sum(counts) belong to no group
    return out


class _GroupedMM(torch.autograd.Function):
    """dX = dY @ w[g]^T per group, dW[g] = X_g^T @ dY_g (layer.py:46-68 of the reference)."""

    @staticmethod
    def forward(ctx, x, w, counts):
        ctx.save_for_backward(x, w, counts)
        return _grouped_mm_plain(x, w, counts)

    @staticmethod
    def backward(ctx, gy):
        x, w, counts = ctx.saved_tensors
        gy = gy.contiguous()
        segs = _segments(counts)
        gx = gy.new_zeros(x.shape)
        gw = torch.zeros_like(w)
        for g, a, b in segs:
            torch.matmul(gy[a:b], w[g].t(), out=gx[a:b])
            gw[g] = x[a:b].t() @ gy[a:b]
        return gx, gw, None


def grouped_mm(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    """Block-diagonal matmul with gradients; on B200 with native ops the tcgen05 grouped GEMM."""
    from . import ops
    if x.is_cuda and ops.custom_ops_enabled() and ops.grouped_supported(x, w):
        return ops.grouped_mm_native(x, w, counts)
    return _GroupedMM.apply(x, w, counts)


def apply_capacity(expert_idx: torch.Tensor, gates: torch.Tensor, n_experts: int,
                   capacity_factor: float | None, n_tokens_global: int | None = None,
                   prior_counts: torch.Tensor | None = None):
    """Capacity-factor token dropping (new capability; the reference is drop-less).

    Every expert accepts at most ``cap = ceil(capacity_factor * T_global * k / E)`` rows.  Rows
    are admitted in canonical order (source rank ascending via ``prior_counts[E]`` = picks of
    lower ranks, then token ascending, then column order); a pick past the cap keeps its slot
    (shapes stay static, "padded") but its gate is zeroed, so it contributes nothing and
    receives no gradient.  Returns ``(gates_kept, keep_mask[T, k], cap)``.
    """
    T, k = expert_idx.shape
    if capacity_factor is None:
        return gates, torch.ones_like(expert_idx, dtype=torch.bool), None
    total = (n_tokens_global if n_tokens_global is not None else T) * k
    cap = int(math.ceil(capacity_factor * total / n_experts))
    flat = expert_idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    sorted_e = flat[order]
    counts = torch.zeros(n_experts, dtype=torch.int64, device=flat.device).scatter_add_(
        0, flat, torch.ones_like(flat))
    starts = torch.cumsum(counts, 0) - counts
    rank_in_e = torch.arange(flat.numel(), device=flat.device) - starts[sorted_e]
    if prior_counts is not None:
        rank_in_e = rank_in_e + prior_counts.to(rank_in_e.dtype)[sorted_e]
    pos = torch.empty_like(rank_in_e)
    pos[order] = rank_in_e
    keep = (pos < cap).view(T, k)
    return gates * keep.to(gates.dtype), keep, cap


class TerracedMoE(nn.Module):
    def __init__(self, hidden: int, d_expert: int, d_shared: int, cfg: TRouteConfig,
                 n_shared: int = 1, bias_gamma: float = 1e-3,
                 capacity_factor: float | None = None):
        super().__init__()
        self.cfg = cfg
        self.bias_gamma = bias_gamma
        self.routing_mode = "full"
        self.expert_backend = "loop"
        self.capacity_factor = capacity_factor
        self.router = Router(hidden, cfg)
        self.shared = SwiGLU(hidden, n_shared * d_shared)
        e = cfg.n_experts
        self.w13 = nn.Parameter(torch.empty(e, hidden, 2 * d_expert))
        self.w2 = nn.Parameter(torch.empty(e, d_expert, hidden))
        nn.init.normal_(self.w13, std=hidden ** -0.5)
        nn.init.normal_(self.w2, std=d_expert ** -0.5)

    # -- routed experts ------------------------------------------------------------------
    def _experts_loop(self, x, expert_idx, gates, y):
        for e in torch.unique(expert_idx).tolist():
            tok, col = (expert_idx == e).nonzero(as_tuple=True)
            gate, up = (x[tok] @ self.w13[e]).chunk(2, dim=-1)
            out = (F.silu(gate) * up) @ self.w2[e]
            y = y.index_add(0, tok, gates[tok, col].unsqueeze(-1).to(out.dtype) * out)
        return y

    def _experts_grouped(self, x, expert_idx, gates, y):
        T, k = expert_idx.shape
        flat_e = expert_idx.reshape(-1)
        order = torch.argsort(flat_e)
        tok = torch.div(order, k, rounding_mode="floor")
        counts = torch.zeros(self.cfg.n_experts, dtype=torch.int64, device=x.device)
        counts.scatter_add_(0, flat_e, torch.ones_like(flat_e))
        gate, up = grouped_mm(x[tok], self.w13, counts).chunk(2, dim=-1)
        out = grouped_mm(F.silu(gate) * up, self.w2, counts)
        w = gates.reshape(-1)[order].unsqueeze(-1).to(out.dtype)
        return y.index_add(0, tok, w * out)

    def _experts_native(self, x, expert_idx, gates, y):
        from . import ops
        return y + ops.moe_experts_local(x, expert_idx, gates, self.w13, self.w2,
                                         self.cfg.group_size)

    def _experts(self, x, expert_idx, gates, y):
        backend = self.expert_backend
        if backend not in EXPERT_BACKENDS:
            raise ValueError(f"unknown expert_backend {backend!r}; expected one of {EXPERT_BACKENDS}")
        if backend == "native":
            return self._experts_native(x, expert_idx, gates, y)
        if backend == "grouped":
            return self._experts_grouped(x, expert_idx, gates, y)
        return self._experts_loop(x, expert_idx, gates, y)

    def forward(self, x: torch.Tensor):
        """x[..., hidden] -> (y of the same shape, stats dict)."""
        lead = x.shape[:-1]
        x = x.reshape(-1, x.shape[-1])
        expert_idx, gates, group_idx = self.router(x, self.routing_mode)
        gates_used, keep, cap = apply_capacity(expert_idx, gates, self.cfg.n_experts,
                                               self.capacity_factor)
        base = self.shared(x)
        y = self._experts(x, expert_idx, gates_used, base)
        load = expert_load(expert_idx, self.cfg.n_experts)
        if self.training:
            update_bias_(self.router.bias, load, self.bias_gamma)
        stats = {"expert_load": load, "group_idx": group_idx, "gates": gates,
                 "expert_idx": expert_idx}
        if cap is not None:
            stats["capacity"] = cap
            stats["dropped"] = (~keep).sum()
        return y.reshape(*lead, -1), stats


class HierarchicalMoE(nn.Module):
    """Terraced compute depth: all tokens through narrow tier-0 experts, the hardest fraction
    ``p`` (lowest top-1 affinity) additionally through wide tier-1 experts, residual-added."""

    def __init__(self, hidden, d0, d1, p, cfg: TRouteConfig, n_shared=1, d_shared=None,
                 bias_gamma=1e-3):
        super().__init__()
        self.p, self.cfg = p, cfg
        self.tier0 = TerracedMoE(hidden, d0, d_shared or 2 * d0, cfg, n_shared=n_shared,
                                 bias_gamma=bias_gamma)
        self.tier1 = TerracedMoE(hidden, d1, d1, cfg, n_shared=0, bias_gamma=bias_gamma)

    @property
    def expert_backend(self):
        return self.tier0.expert_backend

    @expert_backend.setter
    def expert_backend(self, value):
        self.tier0.expert_backend = value
        self.tier1.expert_backend = value

    @property
    def routing_mode(self):
        return self.tier0.routing_mode

    @routing_mode.setter
    def routing_mode(self, value):
        self.tier0.routing_mode = value
        self.tier1.routing_mode = value

    def forward(self, x):
        lead = x.shape[:-1]
        x = x.reshape(-1, x.shape[-1])
        T = x.shape[0]
        mode = self.routing_mode
        aff0 = torch.sigmoid(x @ self.tier0.router.weight.t())
        e0, g0, grp0 = t_route(aff0, self.tier0.router.bias, self.cfg, mode)
        y = self.tier0._experts(x, e0, g0, self.tier0.shared(x))
        n_hard = max(1, int(self.p * T))
        hard = aff0.max(dim=-1).values.argsort()[:n_hard]
        xh = x[hard]
        e1, g1, _ = self.tier1.router(xh, mode)
        yh = self.tier1._experts(xh, e1, g1, torch.zeros_like(xh))
        y = y.index_add(0, hard, yh)
        load0 = expert_load(e0, self.cfg.n_experts)
        if self.training:
            update_bias_(self.tier0.router.bias, load0, self.tier0.bias_gamma)
            update_bias_(self.tier1.router.bias, expert_load(e1, self.cfg.n_experts),
                         self.tier1.bias_gamma)
        stats = {"expert_load": load0, "group_idx": grp0, "gates": g0, "n_hard": n_hard,
                 "expert_idx": e0}
        return y.reshape(*lead, -1), stats
