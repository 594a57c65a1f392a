"""Host-side model of the fused expert-parallel step: placement arithmetic and the flag protocol.

The CUDA kernels of ``ops/csrc/symm.cu`` derive, on every source rank and without any exchange
beyond the per-expert histograms, the row of the OWNER's expert-sorted GEMM input that each
(token, pick) lands in.  This module restates that arithmetic in plain PyTorch for all ranks in
one process, so that it can be checked on a CPU: the positions of all sources must tile every
owner's segments exactly (no gap, no overlap), in (expert, source rank, token) order, with
segments aligned to ``seg_align`` rows.  ``hop_a_rows`` and ``two_hop_model`` do the same for the two-hop path (arrival rows at the
group representatives, forwarding, reduction at the representative and at the origin), and
``return_maps`` / ``scatter_rows`` for the variant in which the GEMM epilogue delivers the output
rows.  It also restates the epoch-flag protocol (flags only grow;
a wait is bounded and returns a status instead of blocking) so that a withheld flag can be tested
without a GPU.

    position(s, t, e) = segment_start(e)                       # owner-local, aligned
                      + sum over sources s' < s of count[s'][e]
                      + number of earlier tokens of source s that picked e

There is no counterpart in the reference (its dispatch is a variable-length collective whose
placement is implied by the split sizes, ``terrace/ep_dist.py:104-122``).
"""
from __future__ import annotations

import torch

ST_OK, ST_TIMEOUT_FLAG, ST_BAD_INDEX, ST_TIMEOUT_COUNTS = 0, 4, 5, 6


def plan_positions(idx_per_rank, world: int, n_experts: int, seg_align: int = 64, cap: int = 0):
    """``idx_per_rank[s]``: ``[T_s, k]`` expert ids of source rank s.  Returns a dict with
    ``pos[s]`` / ``owner[s]`` (``[T_s, k]``), and per owner ``seg_start[o]``, ``seg_count[o]``
    (``[epr]``) and ``rows[o]`` (rows of the owner's buffer in use, padding included).
    ``cap`` > 0: an expert accepts its first ``cap`` rows in (source rank, token) order; the
    picks beyond get position -1 and the segments shrink to ``min(total, cap)``."""
    if len(idx_per_rank) != world or n_experts % world:
        raise ValueError("one index tensor per rank, and world must divide n_experts")
    epr = n_experts // world
    counts = torch.stack([torch.bincount(i.reshape(-1), minlength=n_experts) for i in idx_per_rank])
    before = torch.cumsum(counts, 0) - counts                        # rows of lower sources, [W, E]
    total = counts.sum(0)                                            # [E]
    if cap > 0:
        total = total.clamp(max=cap)
    padded = (total + seg_align - 1) // seg_align * seg_align
    seg = torch.zeros(n_experts, dtype=torch.int64)
    for o in range(world):                                           # owner-local running offset
        block = padded[o * epr:(o + 1) * epr]
        seg[o * epr:(o + 1) * epr] = torch.cumsum(block, 0) - block
    pos, owner = [], []
    for s, idx in enumerate(idx_per_rank):
        T, k = idx.shape
        onehot = torch.zeros(T, n_experts, dtype=torch.int64).scatter_add_(
            1, idx, torch.ones_like(idx))
        if int(onehot.max()) > 1:
            raise ValueError("a token may pick an expert at most once")
        earlier = torch.cumsum(onehot, 0) - onehot                   # earlier tokens picking e
        within = before[s][idx] + earlier.gather(1, idx)             # rank inside the expert
        place = seg[idx] + within
        pos.append(torch.where(within < cap, place, torch.full_like(place, -1)) if cap > 0
                   else place)
        owner.append(torch.div(idx, epr, rounding_mode="floor"))
    return {"pos": pos, "owner": owner,
            "seg_start": [seg[o * epr:(o + 1) * epr].clone() for o in range(world)],
            "seg_count": [total[o * epr:(o + 1) * epr].clone() for o in range(world)],
            "rows": [int(padded[o * epr:(o + 1) * epr].sum()) for o in range(world)]}


def pass1_ranks(idx: torch.Tensor, n_experts: int, chunks: int = 128, lanes: int = 32):
    """The first plan pass as the kernel runs it (``plan_pass1_kernel``): tokens are cut into
    ``chunks`` ranges, a warp walks its range ``lanes`` tokens at a time and ranks every pick
    inside its expert.  Returns ``(es, rank_local, chunk_hist)``: picks sorted ascending per
    token, the rank of each pick among the chunk's picks of the same expert, and the per-chunk
    histogram ``[chunks, E]``.

    For a top-k routing (distinct experts per token) a pick's rank is the count so far plus the
    LOWER lanes of the batch that picked the same expert, whatever their column: token order.
    A batch that holds a token with a repeated expert is ranked column by column instead (still
    distinct, in-range ranks, but not token order)."""
    T, k = idx.shape
    es = torch.sort(idx, dim=1).values
    rank_local = torch.full((T, k), -1, dtype=torch.int64)
    hist = torch.zeros(chunks, n_experts, dtype=torch.int64)
    per = -(-T // chunks) if T else 0
    for c in range(chunks):
        lo, hi = c * per, min(T, (c + 1) * per)
        seen = [0] * n_experts
        for start in range(lo, hi, lanes):
            batch = range(start, min(start + lanes, hi))
            repeated = any(int(es[t, j]) == int(es[t, j - 1]) for t in batch for j in range(1, k))
            if not repeated:
                added = [0] * n_experts
                for t in batch:                                  # lanes ascending = tokens ascending
                    for j in range(k):
                        e = int(es[t, j])
                        if 0 <= e < n_experts:
                            rank_local[t, j] = seen[e] + added[e]
                            added[e] += 1
                seen = [a + b for a, b in zip(seen, added)]
            else:
                for j in range(k):                               # column by column
                    for t in batch:
                        e = int(es[t, j])
                        if 0 <= e < n_experts:
                            rank_local[t, j] = seen[e]
                            seen[e] += 1
        hist[c] = torch.tensor(seen)
    return es, rank_local, hist


def check_tiling(plan, idx_per_rank, world: int, n_experts: int) -> None:
    """Every owner's segment of expert e is covered exactly once, in (source, token) order."""
    epr = n_experts // world
    for o in range(world):
        taken = torch.zeros(max(plan["rows"][o], 1), dtype=torch.int64)
        keys = []                                                    # (row, expert, source, token)
        for s, idx in enumerate(idx_per_rank):
            mine = plan["owner"][s] == o
            rows = plan["pos"][s][mine]
            taken.scatter_add_(0, rows, torch.ones_like(rows))
            tok = torch.arange(idx.shape[0]).unsqueeze(1).expand_as(idx)[mine]
            keys += list(zip(rows.tolist(), idx[mine].tolist(), [s] * rows.numel(), tok.tolist()))
        if int(taken.max()) > 1:
            raise AssertionError(f"owner {o}: two picks share a row")
        for le in range(epr):
            a, n = int(plan["seg_start"][o][le]), int(plan["seg_count"][o][le])
            if n and not bool((taken[a:a + n] == 1).all()):
                raise AssertionError(f"owner {o} expert {o * epr + le}: segment has a gap")
        keys.sort()
        order = [(e, s, t) for _, e, s, t in keys]
        if order != sorted(order):
            raise AssertionError(f"owner {o}: rows are not in (expert, source, token) order")


def return_maps(plan, idx_per_rank, world: int, slots: int):
    """The owners' row maps of the epilogue-push variant: ``map[o][row] = s * slots + t * k + j``
    for the row that source ``s`` pushed for token ``t``'s j-th pick in expert order, ``-1`` for
    padding rows.  The GEMM epilogue stores row ``row`` into rank ``s``'s return slot
    ``t * k + j``."""
    maps = [torch.full((max(plan["rows"][o], 1),), -1, dtype=torch.int64) for o in range(world)]
    for s, idx in enumerate(idx_per_rank):
        T, k = idx.shape
        if T * k > slots:
            raise ValueError("more picks than return slots")
        order = torch.argsort(idx, dim=1, stable=True)
        p_sorted = plan["pos"][s].gather(1, order)
        o_sorted = plan["owner"][s].gather(1, order)
        slot = torch.arange(T * k).view(T, k)
        for o in range(world):
            mine = o_sorted == o
            maps[o][p_sorted[mine]] = s * slots + slot[mine]
    return maps


def scatter_rows(yout, maps, world: int, slots: int, hidden: int, dtype):
    """What the scattering epilogues do, for all owners: every mapped row lands in its origin's
    return section; a map value outside ``[0, world * slots)`` is skipped and counted."""
    ret = [torch.zeros(slots, hidden, dtype=dtype) for _ in range(world)]
    skipped = 0
    for o in range(world):
        m = maps[o]
        rows = torch.nonzero(m != -1).flatten()
        for r in rows.tolist():
            v = int(m[r])
            if v < 0 or v >= world * slots:
                skipped += 1
                continue
            ret[v // slots][v % slots] = yout[o][r]
    return ret, skipped


def one_hop_model(x_per_rank, idx_per_rank, gates_per_rank, w13, w2, group_size: int,
                  seg_align: int = 64, epilogue_push: bool = False):
    """The whole one-hop step on the host: push rows to their positions, grouped SwiGLU per
    segment, pull back and reduce with the canonical tree (per group ascending, one rounding per
    level).  ``w13[E, H, 2d]``, ``w2[E, d, H]`` hold all experts.  Returns ``y`` per rank.
    With ``epilogue_push`` the expert output rows travel through the row maps into the origins'
    return slots and the combine reads those; the reduction order is the same."""
    world, E = len(x_per_rank), w13.shape[0]
    epr = E // world
    plan = plan_positions(idx_per_rank, world, E, seg_align)
    H, dt = x_per_rank[0].shape[1], x_per_rank[0].dtype
    xin = [torch.zeros(max(plan["rows"][o], 1), H, dtype=dt) for o in range(world)]
    for s, x in enumerate(x_per_rank):
        for o in range(world):
            mine = plan["owner"][s] == o
            tok = torch.arange(x.shape[0]).unsqueeze(1).expand_as(mine)[mine]
            xin[o][plan["pos"][s][mine]] = x[tok]
    yout = []
    for o in range(world):
        out = torch.zeros_like(xin[o])
        for le in range(epr):
            a, n = int(plan["seg_start"][o][le]), int(plan["seg_count"][o][le])
            if n:
                gate, up = (xin[o][a:a + n] @ w13[o * epr + le]).chunk(2, dim=-1)
                out[a:a + n] = (torch.nn.functional.silu(gate) * up) @ w2[o * epr + le]
        yout.append(out)
    ret = None
    if epilogue_push:
        slots = max(i.numel() for i in idx_per_rank)
        maps = return_maps(plan, idx_per_rank, world, slots)
        ret, skipped = scatter_rows(yout, maps, world, slots, H, dt)
        if skipped:
            raise AssertionError("a row map entry fell outside the return sections")
    ys = []
    for s, x in enumerate(x_per_rank):
        idx, gates = idx_per_rank[s], gates_per_rank[s]
        order = torch.argsort(idx, dim=1, stable=True)               # experts ascending per token
        e_sorted, g_sorted = idx.gather(1, order), gates.gather(1, order)
        p_sorted, o_sorted = plan["pos"][s].gather(1, order), plan["owner"][s].gather(1, order)
        y = torch.zeros(x.shape[0], H, dtype=torch.float32)
        group = torch.div(e_sorted, group_size, rounding_mode="floor")
        for g in torch.unique(group).tolist():                       # groups ascending
            part = torch.zeros_like(y)
            for j in range(idx.shape[1]):                            # experts ascending inside
                sel = group[:, j] == g
                if not sel.any():
                    rows = None
                elif ret is not None:
                    tok = torch.nonzero(sel).flatten()
                    rows = ret[s][tok * idx.shape[1] + j]
                else:
                    rows = torch.stack([yout[int(o)][int(p)] for o, p in
                                        zip(o_sorted[sel, j], p_sorted[sel, j])])
                if rows is not None:
                    part[sel] += g_sorted[sel, j].float().unsqueeze(1) * rows.float()
            y += part.to(dt).float()                                 # one rounding per level
        ys.append(y.to(dt))
    return ys


def hop_a_rows(idx_per_rank, world: int, n_experts: int, rpn: int, groups_m: int,
               tokens_cap: int):
    """Two-hop, Hop A placement.  Source ``s`` (group ``s // rpn``, local index ``s % rpn``) sends
    one row per (token, run of ``q`` picks in one group ``g``) to the representative
    ``g * rpn + s % rpn``, into row ``(s // rpn) * tokens_cap + rank`` of its arrival section,
    ``rank`` counting the source's earlier items for the same group in (token, run) order.
    Returns per source ``rep[T, M]`` and ``row[T, M]`` (picks sorted by expert first)."""
    epr = n_experts // world
    slots = epr * rpn
    reps, rows = [], []
    for s, idx in enumerate(idx_per_rank):
        T, k = idx.shape
        q = k // groups_m
        es = torch.sort(idx, dim=1).values
        first = es[:, ::q]                                           # first pick of every run
        if not bool((torch.div(es, slots, rounding_mode="floor").view(T, groups_m, q)
                     == torch.div(first, slots, rounding_mode="floor").unsqueeze(2)).all()):
            raise ValueError("a run of q picks spans two groups: routing is not quota-shaped")
        g = torch.div(first, slots, rounding_mode="floor")           # [T, M]
        n_groups = world // rpn
        onehot = torch.nn.functional.one_hot(g.reshape(-1), n_groups)
        rank = (torch.cumsum(onehot, 0) - onehot).gather(1, g.reshape(-1, 1)).view(T, groups_m)
        if int(rank.max()) >= tokens_cap:
            raise ValueError("more Hop A rows for one group than the arrival section holds")
        reps.append(g * rpn + s % rpn)
        rows.append((s // rpn) * tokens_cap + rank)
    return reps, rows


def push_back_rows(rows, reps, rpn: int, tokens_cap: int):
    """Where the reduced (token, group) rows land when the representatives push them back: in
    the origin's own section at ``group * tokens_cap + (arrival row - origin group * tokens_cap)``.
    ``rows`` / ``reps`` as returned by ``hop_a_rows`` for one source; returns ``[T, M]``."""
    origin_group = torch.div(rows, tokens_cap, rounding_mode="floor")
    return torch.div(reps, rpn, rounding_mode="floor") * tokens_cap + (rows - origin_group * tokens_cap)


def two_hop_model(x_per_rank, idx_per_rank, gates_per_rank, w13, w2, rpn: int, groups_m: int,
                  seg_align: int = 64):
    """The two-hop step on the host: Hop A row per (token, group) to the representative, Hop B of
    every pick to its owner at the ORIGIN-computed position (the same positions as one-hop, so
    the expert GEMMs see identical inputs), gate-weighted reduction of the ``q`` picks at the
    representative (fp32, one rounding), sum of the ``M`` group rows at the origin in group order
    (fp32, one rounding).  Returns ``y`` per rank; equals ``one_hop_model`` bit for bit when the
    routing groups are the ``world // rpn`` rank groups."""
    world, E = len(x_per_rank), w13.shape[0]
    epr = E // world
    plan = plan_positions(idx_per_rank, world, E, seg_align)
    H, dt = x_per_rank[0].shape[1], x_per_rank[0].dtype
    cap = max(i.shape[0] for i in idx_per_rank)
    reps, rows = hop_a_rows(idx_per_rank, world, E, rpn, groups_m, cap)
    n_groups = world // rpn
    arrive = [torch.zeros(n_groups * cap, H, dtype=dt) for _ in range(world)]
    used = [torch.zeros(n_groups * cap, dtype=torch.int64) for _ in range(world)]
    for s, x in enumerate(x_per_rank):                               # Hop A
        for m in range(groups_m):
            for t in range(x.shape[0]):
                r, a = int(reps[s][t, m]), int(rows[s][t, m])
                arrive[r][a] = x[t]
                used[r][a] += 1
    if any(int(u.max()) > 1 for u in used):
        raise AssertionError("two Hop A rows share an arrival slot")
    xin = [torch.zeros(max(plan["rows"][o], 1), H, dtype=dt) for o in range(world)]
    order = [torch.argsort(i, dim=1, stable=True) for i in idx_per_rank]
    for s, idx in enumerate(idx_per_rank):                           # Hop B, from the arrival rows
        k = idx.shape[1]
        q = k // groups_m
        p_sorted = plan["pos"][s].gather(1, order[s])
        o_sorted = plan["owner"][s].gather(1, order[s])
        for t in range(idx.shape[0]):
            for j in range(k):
                m = j // q
                src = arrive[int(reps[s][t, m])][int(rows[s][t, m])]
                xin[int(o_sorted[t, j])][int(p_sorted[t, j])] = src
    yout = []
    for o in range(world):
        out = torch.zeros_like(xin[o])
        for le in range(epr):
            a, n = int(plan["seg_start"][o][le]), int(plan["seg_count"][o][le])
            if n:
                gate, up = (xin[o][a:a + n] @ w13[o * epr + le]).chunk(2, dim=-1)
                out[a:a + n] = (torch.nn.functional.silu(gate) * up) @ w2[o * epr + le]
        yout.append(out)
    ys = []
    for s, x in enumerate(x_per_rank):
        idx, gates = idx_per_rank[s], gates_per_rank[s]
        k = idx.shape[1]
        q = k // groups_m
        g_sorted = gates.gather(1, order[s])
        p_sorted = plan["pos"][s].gather(1, order[s])
        o_sorted = plan["owner"][s].gather(1, order[s])
        y = torch.zeros(x.shape[0], H, dtype=torch.float32)
        for m in range(groups_m):                                    # groups ascending
            red = torch.zeros(x.shape[0], H, dtype=torch.float32)
            for j in range(m * q, (m + 1) * q):                      # at the representative
                rows_j = torch.stack([yout[int(o)][int(p)] for o, p in
                                      zip(o_sorted[:, j], p_sorted[:, j])])
                red += g_sorted[:, j].float().unsqueeze(1) * rows_j.float()
            y += red.to(dt).float()                                  # the reduced row travels as bf16
        ys.append(y.to(dt))
    return ys


class EpochFlags:
    """Flags of one arena: ``flag[kind][src]`` holds the last epoch that source signalled.
    ``signal`` never lowers a flag; ``wait`` polls a bounded number of times and returns a status
    code (``ST_OK`` or the timeout code) instead of blocking."""

    def __init__(self, kinds: int, world: int):
        self.flags = [[0] * world for _ in range(kinds)]

    def signal(self, kind: int, src: int, epoch: int) -> None:
        self.flags[kind][src] = max(self.flags[kind][src], epoch)

    def wait(self, kind: int, sources, epoch: int, max_polls: int = 1000,
             timeout_code: int = ST_TIMEOUT_FLAG, on_poll=None) -> int:
        for _ in range(max_polls):
            if all(self.flags[kind][s] >= epoch for s in sources):
                return ST_OK
            if on_poll is not None:
                on_poll()
        return timeout_code
