"""T-A2A: two-hop expert-parallel dispatch/combine over ``torch.distributed`` (closed forward).

Hop A sends ONE row per (token, destination group) to the group representative
``group*rpn + (rank % rpn)``; the arrival rank expands each row into its (row, expert-slot)
pairs, bucket-sorts them by owner rank inside the group, and Hop B delivers each pair to the
rank that owns the expert.  The return leg reverses Hop B, applies the gate AT THE ARRIVAL
RANK while reducing the q pairs of a row, reverses Hop A and sums a token's M group rows.

Parity with the reference ``terrace/ta2a_fwd.py``:
  * ``init_ta2a_groups``                       -> ta2a_fwd.py:269-296
  * ``fixed_hist``                             -> ta2a_fwd.py:299-321
  * ``build_expansion`` (int64 slot bitmask)   -> ta2a_fwd.py:348-442
  * quota wire format ``[S,q]`` slots + gates  -> ta2a_fwd.py:177-249
  * arrival expansion                          -> ta2a_fwd.py:120-174, 252-266
  * ``ta2a_moe_forward``                       -> ta2a_fwd.py:445-670
  * gate-at-arrival                            -> ta2a_fwd.py:500-517

Differences by design: slot ids are plain integers (no 63-slot bound on the quota path); an
origin key ``(source rank, token)`` rides in the integer planes so the expert GEMM sees rows in
the canonical (expert, source rank, token) order and the result is bit-identical to the
one-hop path (see ``parallel/ep.py``); counts use integer scans.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from ..ops.refs import fixed_hist, stable_bucket_order
from .ep import (CALLS, _a2a, _a2a_raw, ep_moe_forward, exchange_counts, sort_picks,
                 swiglu_experts)
from .plan import plan_ta2a

_GROUPS: dict = {}
KEY_SHIFT = 32

CALLS.setdefault("two_hop", 0)


def init_ta2a_groups(world: int, rpn: int = 8):
    """Create (once per ``(world, rpn)``) the intra-group communicators ``{g*rpn .. g*rpn+rpn-1}``
    and the inter-group communicators ``{l, l+rpn, ...}``.  Collective over the world: every
    rank must call it, in the same order, before the first forward.  Returns this rank's
    intra-group communicator."""
    if world % rpn:
        raise ValueError(f"world={world} is not a multiple of rpn={rpn}")
    key = (world, rpn)
    if key not in _GROUPS:
        rank = dist.get_rank()
        intra = inter = None
        for g in range(world // rpn):
            members = list(range(g * rpn, (g + 1) * rpn))
            grp = dist.new_group(members)
            if rank in members:
                intra = grp
        for l in range(rpn):
            members = list(range(l, world, rpn))
            grp = dist.new_group(members)
            if rank in members:
                inter = grp
        _GROUPS[key] = (intra, inter)
    return _GROUPS[key][0]


def get_ta2a_groups(world: int, rpn: int):
    if (world, rpn) not in _GROUPS:
        raise RuntimeError("init_ta2a_groups(world, rpn) must run on every rank before the "
                           "first T-A2A forward")
    return _GROUPS[(world, rpn)]


def reset_groups() -> None:
    _GROUPS.clear()


def build_expansion(expert_idx, inverse, n_rows: int, world: int, n_experts: int, rpn: int = 8,
                    groups_m: int | None = None, *, sorted_rows: bool = False, slot_flat=None):
    """int64 bitmask per send row: bit j set iff the row's token wants slot j of that group.
    Only defined for at most 63 slots per group (the general, non-quota wire format)."""
    slots = (n_experts // world) * rpn
    if slots > 63:
        raise ValueError(f"{slots} expert slots per group do not fit the int64 bitmask; use the "
                         f"quota wire format (pass groups_m)")
    if slot_flat is None:
        slot_flat = (expert_idx % slots).reshape(-1)
    bits = torch.ones_like(slot_flat) << slot_flat
    mask = torch.zeros(n_rows, dtype=torch.int64, device=expert_idx.device)
    return mask.scatter_add_(0, inverse, bits)          # picks of a row are distinct: add == or


def pack_quota_wire(e_sorted, g_sorted, inverse_sorted, n_rows: int, slots: int, q: int):
    """Quota wire format.  Inputs are per-token ascending; returns ``slot_tab[S,q]`` (ascending
    slot ids) and ``gate_tab[S,q]`` (co-indexed gates, differentiable w.r.t. ``g_sorted``)."""
    T, k = e_sorted.shape
    m = k // q
    rows = inverse_sorted.view(T, m, q)[:, :, 0].reshape(-1)               # row of (t, j-th group)
    slot_tab = torch.zeros(n_rows, q, dtype=torch.int64, device=e_sorted.device)
    slot_tab.index_copy_(0, rows, (e_sorted % slots).view(T * m, q))
    gate_tab = g_sorted.new_zeros(n_rows, q).index_copy(0, rows, g_sorted.reshape(T * m, q))
    return slot_tab, gate_tab, rows.view(T, m)


def expand_arrival_mask(rmask: torch.Tensor, slots: int):
    """Bitmask rows -> (r_idx, slot_idx) row-major, slot ascending (host sync for the size)."""
    bits = (rmask.unsqueeze(1) >> torch.arange(slots, device=rmask.device)) & 1
    r_idx, slot_idx = bits.nonzero(as_tuple=True)
    return r_idx, slot_idx


class _RowGather(torch.autograd.Function):
    """``x[u_src]``; gradient added per token in send-row order (group ascending) in fp32."""

    @staticmethod
    def forward(ctx, x, u_src):
        ctx.save_for_backward(u_src)
        ctx.shape = tuple(x.shape)
        return x[u_src]

    @staticmethod
    def backward(ctx, g):
        (u_src,) = ctx.saved_tensors
        acc = torch.zeros(ctx.shape, dtype=torch.float32, device=g.device)
        acc.index_add_(0, u_src, g.float())
        return acc.to(g.dtype), None


def ta2a_moe_forward(x_local, expert_idx, gates, w13_shard, w2_shard, world: int, n_experts: int,
                     rpn: int = 8, groups_m: int | None = None, *, canonical: bool = True,
                     experts_fn=None):
    """Routed-expert output for this rank's tokens under two-hop EP.

    ``groups_m=M`` declares equal-quota routing (exactly ``k/M`` picks in each of M groups per
    token): static shapes and the quota wire format.  ``None`` takes the general bitmask format
    (host syncs, at most 63 slots per group).  Fewer than two groups falls back to one-hop.
    """
    n_nodes = world // rpn
    if n_nodes < 2:
        return ep_moe_forward(x_local, expert_idx, gates, w13_shard, w2_shard, world, n_experts,
                              rpn=rpn, canonical=canonical, experts_fn=experts_fn)
    CALLS["two_hop"] += 1
    intra, _inter = get_ta2a_groups(world, rpn)
    rank = dist.get_rank()
    my_local = rank % rpn
    epr = n_experts // world
    slots = epr * rpn
    T, k = expert_idx.shape
    H = x_local.shape[1]
    dev = x_local.device
    dt = x_local.dtype

    e_sorted, g_sorted, _ = sort_picks(expert_idx, gates)
    u_src, u_node, counts, inverse = plan_ta2a(e_sorted, world, n_experts, rpn, groups_m)
    n_rows = u_src.shape[0]
    payload = _RowGather.apply(x_local, u_src)
    key = (torch.full_like(u_src, rank) << KEY_SHIFT) | u_src
    if groups_m is not None:
        q = k // groups_m
        slot_tab, gate_tab, rows_tm = pack_quota_wire(e_sorted, g_sorted, inverse, n_rows, slots, q)
        ids = torch.cat([slot_tab, key.unsqueeze(1)], dim=1)              # [S, q+1]
    else:
        q = None
        slot_flat = (e_sorted % slots).reshape(-1)
        mask = build_expansion(e_sorted, inverse, n_rows, world, n_experts, rpn,
                               slot_flat=slot_flat)
        gate_tab = g_sorted.new_zeros(n_rows, slots).index_put(
            (inverse, slot_flat), g_sorted.reshape(-1))
        ids = torch.stack([mask, key], dim=1)                              # [S, 2]

    # ---- Hop A: world all-to-all with N_g non-zero splits (to each group's representative)
    send = torch.zeros(world, dtype=torch.int64, device=dev)
    send[torch.arange(n_nodes, device=dev) * rpn + my_local] = counts
    recv = exchange_counts(send)
    send_l, recv_l = send.tolist(), recv.tolist()
    rx = _a2a(payload, send_l, recv_l)
    rids = _a2a_raw(ids, send_l, recv_l)
    rgate = _a2a(gate_tab, send_l, recv_l)                               # differentiable

    # ---- arrival chain
    R = rx.shape[0]
    if q is not None:
        rslot, rkey = rids[:, :q].contiguous(), rids[:, q]
        send_buf, gate_pairs, r_idx, slot_idx, i_send = ops.k1_arrival(
            rx, rslot, rgate, q, epr, rpn, my_local)
        order_pairs = None
    else:
        rmask, rkey = rids[:, 0], rids[:, 1]
        r0, s0 = expand_arrival_mask(rmask, slots)
        owner = torch.div(s0, epr, rounding_mode="floor")
        order_pairs = stable_bucket_order(owner, rpn)
        r_idx, slot_idx = r0[order_pairs], s0[order_pairs]
        i_send = fixed_hist(owner, rpn)
        send_buf = _RowGather.apply(rx, r_idx)
        gate_pairs = rgate[r_idx, slot_idx]
    key_pairs = rkey[r_idx]

    # ---- Hop B: intra-group, demand sized
    i_recv = exchange_counts(i_send, intra)
    is_l, ir_l = i_send.tolist(), i_recv.tolist()
    node_rx = _a2a(send_buf, is_l, ir_l, intra)
    meta = _a2a_raw(torch.stack([slot_idx, key_pairs], dim=1), is_l, ir_l, intra)
    exp_j = meta[:, 0] - my_local * epr
    if canonical:
        by_key = torch.argsort(meta[:, 1], stable=True)
        order = by_key[torch.argsort(exp_j[by_key], stable=True)]         # (expert, src, token)
    else:
        order = torch.argsort(exp_j, stable=True)
    tokens_per_expert = fixed_hist(exp_j, epr)
    ye = (experts_fn or swiglu_experts)(node_rx[order], w13_shard, w2_shard, tokens_per_expert)
    unsort = torch.empty_like(order)
    unsort[order] = torch.arange(order.numel(), device=dev)

    # ---- combine: reverse Hop B, gate-weighted reduce at the arrival rank, reverse Hop A
    ret = _a2a(ye[unsort], ir_l, is_l, intra)
    weighted = ret.float() * gate_pairs.unsqueeze(-1).float()
    if q is not None and canonical:
        owner = torch.div(rslot.reshape(-1), epr, rounding_mode="floor")
        place = stable_bucket_order(owner, rpn)                            # pair -> r*q + i
        by_row = torch.zeros(R * q, H, dtype=torch.float32, device=dev).index_copy(
            0, place, weighted).view(R, q, H)
        red32 = torch.zeros(R, H, dtype=torch.float32, device=dev)
        for i in range(q):
            red32 = red32 + by_row[:, i]
    else:
        red32 = torch.zeros(R, H, dtype=torch.float32, device=dev).index_add(0, r_idx, weighted)
    red = red32.to(dt)
    back = _a2a(red, recv_l, send_l)
    if q is not None and canonical:
        y32 = torch.zeros(T, H, dtype=torch.float32, device=dev)
        for m in range(groups_m):
            y32 = y32 + back[rows_tm[:, m]].float()
    else:
        y32 = torch.zeros(T, H, dtype=torch.float32, device=dev).index_add(0, u_src, back.float())
    return y32.to(dt)
