"""Executable PyTorch specifications of the fused index kernels (CPU and GPU).

  * ``fixed_hist``            fixed-length histogram without a host sync
                              (reference ``terrace/ta2a_fwd.py:299-321``)
  * ``stable_bucket_order``   stable ascending argsort of small integer keys
                              (reference ``terrace/ta2a_fwd.py:324-345``; plain integer sort here)
  * ``k1_arrival_ref``        arrival chain: expand (row, slot) pairs, stable bucket sort by
                              owner rank, gather rows and gates
                              (reference ``terrace/ops/__init__.py:255-300``)
  * ``k2_pack_ref``           send-side pack: per-token ascending sort, one row per
                              (token, group) in (group asc, token asc) order
                              (reference ``terrace/ops/k2_ref.py:70-134``)

The CUDA kernels are tested bit-for-bit against these functions.  Unlike the reference there
is no 63-slot bound: slot ids travel as integers, not as an int64 bitmask.
"""
from __future__ import annotations

import torch


def fixed_hist(idx: torch.Tensor, n_buckets: int) -> torch.Tensor:
    out = torch.zeros(n_buckets, dtype=torch.int64, device=idx.device)
    flat = idx.reshape(-1).to(torch.int64)
    if flat.numel():
        out.scatter_add_(0, flat, torch.ones_like(flat))
    return out


def stable_bucket_order(key: torch.Tensor, n_buckets: int) -> torch.Tensor:
    """Permutation that sorts ``key`` (values in ``[0, n_buckets)``) ascending, ties in index
    order.  Composite integer key ``key * n + position`` makes the order total, so a plain
    (unstable) sort suffices."""
    n = key.numel()
    if n == 0:
        return torch.zeros(0, dtype=torch.int64, device=key.device)
    comp = key.to(torch.int64) * n + torch.arange(n, device=key.device, dtype=torch.int64)
    return torch.argsort(comp)


def k1_arrival_ref(rx: torch.Tensor, rslot: torch.Tensor, rgate: torch.Tensor, quota: int,
                   epr: int, rpn: int, my_local: int = 0):
    """``(rx[R,H], rslot[R,q] int64 ascending, rgate[R,q]) -> (send_buf[R*q,H], gate_pairs[R*q],
    r_idx[R*q], slot_idx[R*q], i_send[rpn])`` in (owner asc, row asc, slot asc) order.
    ``my_local`` is part of the interface (the kernel carries it) and unused by this segment."""
    R, q = rslot.shape
    if q != quota:
        raise AssertionError(f"rslot has {q} columns but quota is {quota}")
    flat = rslot.reshape(-1)
    owner = torch.div(flat, epr, rounding_mode="floor")
    order = stable_bucket_order(owner, rpn)
    r_idx = torch.div(order, quota, rounding_mode="floor")
    return (rx[r_idx], rgate.reshape(-1)[order], r_idx, flat[order], fixed_hist(owner, rpn))


def k2_pack_ref(hidden: torch.Tensor, expert_idx: torch.Tensor, gates: torch.Tensor, world: int,
                n_experts: int, rpn: int, groups_m: int, *, max_slots: int | None = None):
    """``(hidden[T,H], expert_idx[T,k], gates[T,k]) -> (payload[T*M,H], mask[T*M,q] ascending
    slot ids, gate_rows[T*M,q], u_src[T*M], node_counts[N_g])``; rows ordered (group asc,
    token asc).  Requires equal-quota routing (exactly q picks in each of M groups per token)."""
    if hidden.dim() != 2 or expert_idx.dim() != 2 or gates.dim() != 2:
        raise ValueError("k2_pack: hidden, expert_idx and gates must be 2-D")
    T, k = expert_idx.shape
    if hidden.shape[0] != T or gates.shape != expert_idx.shape:
        raise ValueError(f"k2_pack: geometry mismatch hidden={tuple(hidden.shape)} "
                         f"expert_idx={tuple(expert_idx.shape)} gates={tuple(gates.shape)}")
    if gates.dtype != hidden.dtype:
        raise RuntimeError(f"k2_pack: gates dtype {gates.dtype} != hidden dtype {hidden.dtype}; "
                           f"cast at the caller, who owns the rounding point")
    if min(world, rpn, groups_m, n_experts) <= 0:
        raise ValueError("k2_pack: geometry scalars must be positive")
    if world % rpn or n_experts % world or k % groups_m:
        raise ValueError(f"k2_pack: world={world} rpn={rpn} n_experts={n_experts} k={k} "
                         f"groups_m={groups_m} do not divide")
    slots = (n_experts // world) * rpn
    n_nodes = world // rpn
    q = k // groups_m
    if max_slots is not None and slots > max_slots:
        raise ValueError(f"{slots} expert slots per group exceeds the bound {max_slots}")
    if T and (int(expert_idx.min()) < 0 or int(expert_idx.max()) >= n_experts):
        raise ValueError("k2_pack: expert id out of range")
    P = T * groups_m
    e_sorted, cols = torch.sort(expert_idx, dim=1, stable=True)
    g_sorted = gates.gather(1, cols)
    dest = torch.div(e_sorted[:, ::q], slots, rounding_mode="floor").reshape(-1)      # [T*M]
    order = stable_bucket_order(dest, n_nodes)
    u_src = torch.div(order, groups_m, rounding_mode="floor")
    mask = (e_sorted % slots).reshape(P, q)[order]
    gate_rows = g_sorted.reshape(P, q)[order]
    return hidden[u_src], mask, gate_rows, u_src, fixed_hist(dest, n_nodes)
