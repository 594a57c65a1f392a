"""One-hop expert parallelism over ``torch.distributed`` (the baseline arm and the CPU/gloo
plumbing path) plus the differentiable all-to-all primitives every EP path shares.

Parity with the reference ``terrace/ep_dist.py``:
  * ``_a2a_raw`` (splits as lists or tensors)        -> ep_dist.py:17-37
  * ``_A2A`` (backward = transpose exchange, same group) -> ep_dist.py:40-67
  * ``_a2a`` (autograd for floats, raw for ints)      -> ep_dist.py:70-79
  * ``ep_moe_forward``                                -> ep_dist.py:82-122

Canonical arithmetic (shared with the two-hop path so the two are bit-identical, forward and
backward):
  * expert GEMM rows are ordered (expert asc, source rank asc, token asc);
  * a token's output is ``sum over groups asc ( sum over experts asc in group gate*out )``,
    every level accumulated left to right in fp32 from zero, a group partial rounded once to
    the payload dtype (it is the value that crosses the fabric on the two-hop return leg);
  * the gradient of a token's row uses the same tree.
``canonical=False`` restores the reference's flat ``index_add`` over the k picks.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..layer import grouped_mm

# Live-path counters: tests read these to prove which path ran.
CALLS = {"a2a": 0, "a2a_autograd": 0, "one_hop": 0}


def _as_list(splits):
    return splits.tolist() if torch.is_tensor(splits) else list(splits)


def _a2a_raw(x: torch.Tensor, in_splits, out_splits, group=None) -> torch.Tensor:
    """Variable-split all-to-all along dim 0; ``in_splits``/``out_splits`` lists or tensors."""
    in_l, out_l = _as_list(in_splits), _as_list(out_splits)
    out = x.new_empty((sum(out_l), *x.shape[1:]))
    CALLS["a2a"] += 1
    dist.all_to_all_single(out, x.contiguous(), out_l, in_l, group=group)
    return out


class _A2A(torch.autograd.Function):
    """Differentiable all-to-all: the adjoint is the same exchange with the splits swapped,
    on the same process group."""

    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group=None):
        ctx.in_l, ctx.out_l, ctx.group = _as_list(in_splits), _as_list(out_splits), group
        CALLS["a2a_autograd"] += 1
        return _a2a_raw(x, ctx.in_l, ctx.out_l, group)

    @staticmethod
    def backward(ctx, g):
        return _a2a_raw(g, ctx.out_l, ctx.in_l, ctx.group), None, None, None


def _a2a(x, in_splits, out_splits, group=None):
    if x.is_floating_point() and torch.is_grad_enabled():
        return _A2A.apply(x, in_splits, out_splits, group)
    return _a2a_raw(x, in_splits, out_splits, group)


def exchange_counts(send: torch.Tensor, group=None) -> torch.Tensor:
    """Counts all-to-all: element i of ``send`` goes to rank i; returns what every rank sent us."""
    recv = torch.empty_like(send)
    CALLS["a2a"] += 1
    dist.all_to_all_single(recv, send, group=group)
    return recv


def hist(idx: torch.Tensor, n: int) -> torch.Tensor:
    """Fixed-length int64 histogram without a host sync (``bincount`` syncs to size its output)."""
    out = torch.zeros(n, dtype=torch.int64, device=idx.device)
    if idx.numel():
        out.scatter_add_(0, idx.reshape(-1).long(), torch.ones(idx.numel(), dtype=torch.int64,
                                                               device=idx.device))
    return out


# ---------------------------------------------------------------------------------------------
# canonical reduction tree
# ---------------------------------------------------------------------------------------------
def nested_reduce(rows: torch.Tensor, gid: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """``rows[T, k, H]`` whose k columns are ordered by ascending expert id, ``gid[T, k]`` the
    group of every column.  Returns ``[T, H]``: within a group left-to-right fp32 sums from
    zero, the partial rounded to ``out_dtype``, partials added left to right in fp32 from zero,
    the total rounded to ``out_dtype``.  Built from differentiable ops (the adjoint is a plain
    broadcast, so no reduction order is involved in its backward)."""
    T, k, H = rows.shape
    out_dtype = out_dtype or rows.dtype
    total = torch.zeros(T, H, dtype=torch.float32, device=rows.device)
    partial = torch.zeros(T, H, dtype=torch.float32, device=rows.device)
    for j in range(k):
        if j > 0:
            fresh = (gid[:, j] != gid[:, j - 1]).unsqueeze(-1)
            flushed = total + partial.to(out_dtype).float()
            total = torch.where(fresh, flushed, total)
            partial = torch.where(fresh, torch.zeros_like(partial), partial)
        partial = partial + rows[:, j].float()
    total = total + partial.to(out_dtype).float()
    return total.to(out_dtype)


class _PairExpand(torch.autograd.Function):
    """``x[T, H] -> [T, k, H]`` (one copy per pick); the gradient folds the k copies back with
    :func:`nested_reduce`, i.e. the same tree the two-hop path applies hop by hop."""

    @staticmethod
    def forward(ctx, x, gid):
        ctx.save_for_backward(gid)
        return x.unsqueeze(1).expand(x.shape[0], gid.shape[1], x.shape[1]).contiguous()

    @staticmethod
    def backward(ctx, g):
        (gid,) = ctx.saved_tensors
        return nested_reduce(g, gid, g.dtype), None


def sort_picks(expert_idx: torch.Tensor, gates: torch.Tensor):
    """Order every token's picks by ascending expert id (gates follow)."""
    e_sorted, cols = torch.sort(expert_idx, dim=1, stable=True)
    return e_sorted, gates.gather(1, cols), cols


def swiglu_experts(rows: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, counts: torch.Tensor):
    gate, up = grouped_mm(rows, w13, counts).chunk(2, dim=-1)
    return grouped_mm(F.silu(gate) * up, w2, counts)


def ep_moe_forward(x_local: torch.Tensor, expert_idx: torch.Tensor, gates: torch.Tensor,
                   w13_shard: torch.Tensor, w2_shard: torch.Tensor, world: int, n_experts: int,
                   *, group=None, rpn: int | None = None, canonical: bool = True,
                   experts_fn=None) -> torch.Tensor:
    """Routed-expert output for this rank's tokens under one-hop EP (4 collectives forward).

    Rank r owns experts ``[r*epr, (r+1)*epr)``.  ``rpn`` (ranks per logical group) only
    selects the grouping of the canonical reduction tree; ``None`` means a single group.
    ``experts_fn(rows, w13, w2, counts)`` replaces the expert compute (default: the SwiGLU
    experts); a benchmark passes the identity to time the exchange alone.
    """
    CALLS["one_hop"] += 1
    if n_experts % world:
        raise ValueError(f"n_experts={n_experts} is not divisible by world={world}")
    epr = n_experts // world
    T, k = expert_idx.shape
    H = x_local.shape[1]
    dev = x_local.device
    slots = epr * (rpn if rpn else world)

    if canonical:
        e_sorted, g_sorted, _ = sort_picks(expert_idx, gates)
        gid = torch.div(e_sorted, slots, rounding_mode="floor")
        pairs = _PairExpand.apply(x_local, gid).reshape(T * k, H)
    else:
        e_sorted, g_sorted = expert_idx, gates
        pairs = x_local.repeat_interleave(k, dim=0)
    eid = e_sorted.reshape(-1)
    dest = torch.div(eid, epr, rounding_mode="floor")
    perm = torch.argsort(dest, stable=True)
    send = hist(dest, world)
    recv = exchange_counts(send, group)
    send_l, recv_l = send.tolist(), recv.tolist()

    rx = _a2a(pairs[perm], send_l, recv_l, group)
    reid = _a2a((eid[perm] % epr).to(torch.int32), send_l, recv_l, group).long()

    order = torch.argsort(reid, stable=True)            # (expert, source rank, token)
    counts = hist(reid, epr)
    ye = (experts_fn or swiglu_experts)(rx[order], w13_shard, w2_shard, counts)
    unsort = torch.empty_like(order)
    unsort[order] = torch.arange(order.numel(), device=dev)
    back = _a2a(ye[unsort], recv_l, send_l, group)

    inv_perm = torch.empty_like(perm)
    inv_perm[perm] = torch.arange(perm.numel(), device=dev)
    out_pairs = back[inv_perm].view(T, k, H)
    if canonical:
        weighted = out_pairs.float() * g_sorted.unsqueeze(-1).float()
        return nested_reduce(weighted, gid, x_local.dtype)
    y = x_local.new_zeros(T, H)
    tok = torch.arange(T, device=dev).repeat_interleave(k)
    return y.index_add(0, tok[perm], (g_sorted.reshape(-1)[perm].unsqueeze(-1).to(back.dtype)
                                      * back))
