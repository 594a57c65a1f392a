"""T-A2A send plan: one row per distinct (token, destination group), group-major.

Parity with the reference ``terrace/ta2a.py``:
  * ``plan_ta2a`` (returns ``u_src, u_node, counts, inverse``; ``groups_m`` fast path with a
    static row count ``T*M`` and a fan-out/quota verification on the first call and every
    256th per shape key)                               -> ta2a.py:70-275
  * ``dispatch_stats`` ledger                          -> ta2a.py:278-298

The reference builds the plan from float32 scans and float-key sorts because integer scans
were slow on its accelerator; here plain int64 ``cumsum``/``searchsorted`` are used, so there
is no 2^24 bound.  Row order (group ascending, token ascending) is part of the contract: it
fixes every downstream reduction order.
"""
from __future__ import annotations

import torch

VERIFY_EVERY = 256
_VERIFIED: set = set()
_VERIFY_CALLS: dict = {}
_VERIFY_COUNT = _VERIFY_CALLS          # the name the reference's tests clear


def reset_plan_cache() -> None:
    _VERIFIED.clear()
    _VERIFY_CALLS.clear()


def _verify_quota(occ: torch.Tensor, dest: torch.Tensor, T: int, k: int, groups_m: int) -> None:
    """Host-synchronising check of both halves of the equal-quota invariant."""
    n_rows = T * groups_m
    actual = int(occ.sum().item())
    if actual != n_rows:
        raise ValueError(
            f"groups_m={groups_m} implies {n_rows} send rows for T={T}, but the routing produces "
            f"{actual} (fan-out {actual / max(T, 1):.4f} != {groups_m}); pass groups_m only for "
            f"routings with an exact fan-out")
    per = torch.zeros(occ.shape, dtype=torch.int64, device=occ.device)
    per.scatter_add_(1, dest, torch.ones_like(dest))
    bad = int(((per > 0) & (per != k // groups_m)).sum().item())
    if bad:
        raise ValueError(
            f"groups_m={groups_m} needs every touched group to hold exactly k/M={k // groups_m} "
            f"of a token's experts, but {bad} (token, group) pairs break the quota; this routing "
            f"is not equal-quota -- leave groups_m None")


def plan_ta2a(expert_idx: torch.Tensor, world: int, n_experts: int, rpn: int = 8,
              groups_m: int | None = None):
    """``expert_idx[T, k]`` -> ``(u_src[S], u_node[S], counts[N_g], inverse[T*k])``.

    ``u_src`` token of every send row, ``u_node`` its destination group (ascending),
    ``counts`` rows per group, ``inverse`` the send row that carries pick ``(t, j)``.
    With ``groups_m=M`` the row count is the static ``T*M`` and no host sync happens outside
    the periodic verification; with ``None`` the count is read back from the device.
    """
    if world % rpn or n_experts % world:
        raise ValueError(f"world={world}, rpn={rpn}, n_experts={n_experts} do not divide")
    slots = (n_experts // world) * rpn
    n_nodes = world // rpn
    T, k = expert_idx.shape
    dev = expert_idx.device
    dest = torch.div(expert_idx, slots, rounding_mode="floor")            # [T, k]
    occ = torch.zeros(T, n_nodes, dtype=torch.bool, device=dev)
    occ.scatter_(1, dest, True)
    node_major = occ.t().reshape(-1)                                      # [N_g * T]
    running = torch.cumsum(node_major.to(torch.int64), 0)                 # inclusive

    if groups_m is None:
        sel = node_major.nonzero(as_tuple=False).reshape(-1)              # host sync (size)
    else:
        if k % groups_m:
            raise ValueError(f"groups_m={groups_m} does not divide k={k}: the per-group quota "
                             f"is not an integer")
        key = (T, k, n_nodes, groups_m)
        calls = _VERIFY_CALLS.get(key, 0)
        _VERIFY_CALLS[key] = calls + 1
        if key not in _VERIFIED or calls % VERIFY_EVERY == 0:
            _verify_quota(occ, dest, T, k, groups_m)
            _VERIFIED.add(key)
        want = torch.arange(T * groups_m, device=dev, dtype=torch.int64)
        sel = torch.searchsorted(running, want, right=True)
    u_node = torch.div(sel, max(T, 1), rounding_mode="floor")
    u_src = sel - u_node * T
    counts = occ.sum(dim=0, dtype=torch.int64)
    flat = dest * T + torch.arange(T, device=dev, dtype=dest.dtype).unsqueeze(1)
    inverse = (running - 1)[flat.reshape(-1)]
    return u_src, u_node, counts, inverse


def dispatch_stats(expert_idx: torch.Tensor, world: int, n_experts: int, rpn: int = 8) -> dict:
    """Rows/messages of one dispatch: per-pick baseline against per-(token, group) T-A2A."""
    T, k = expert_idx.shape
    _, _, counts, _ = plan_ta2a(expert_idx, world, n_experts, rpn)
    rows = int(counts.sum())
    return {
        "rows_baseline": T * k,
        "rows_ta2a": rows,
        "dedup_x": (T * k) / max(rows, 1),
        "msgs_baseline": world,
        "msgs_ta2a": world // rpn,
        "msg_growth_x": rpn,
    }
