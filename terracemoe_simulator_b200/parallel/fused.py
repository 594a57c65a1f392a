"""Fused expert parallelism over peer memory: the product path for dispatch / combine.

``FusedEPContext`` owns one symmetric arena per MoE layer (see ``ops/csrc/symm_layout.h``): every
rank ``cudaMalloc``s the same layout, exports it with CUDA IPC, and maps all peers.  The kernels
(``ops/csrc/symm.cu``) then move token rows with plain peer stores/loads and synchronise with
epoch flags; NCCL is used only to exchange the IPC handles at start-up.

One step of ``fused_moe_forward`` (no host synchronisation anywhere):

  one-hop   plan -> push rows into the owners' expert-sorted input -> [GEMM1 waits on the
            arrival flags of its A operand] SwiGLU GEMMs -> signal -> gate-weighted pull combine
  two-hop   plan -> Hop A push (one row per (token, group) + header) to the representative ->
            representative forwards every (row, pick) to the owner (Hop B) -> GEMMs -> the
            representative pulls, applies the gates and reduces per row -> origin pulls and adds
            its M group rows

Two-hop with ``TERRACE_EP_PUSH_BACK=1`` (off by default): the representative stores each reduced
(token, group) row into the ORIGIN's section (block of the representative's group, same row
inside the block) instead of keeping it for the origin to read remotely; the origin's final sum
then reads local memory.  Values and order are unchanged.

One-hop with ``epilogue_push`` (``TERRACE_EP_EPILOGUE_PUSH=1``; off by default): the push also
leaves every row's return address in the owner's row map, the second expert GEMM stores each
output row from its epilogue straight into the ORIGIN's return slot over NVLink (one kernel does
the GEMM and the combine transfer, tile by tile), and the combine reads local memory only.  The
reduction order is unchanged, so the result equals the pull path bit for bit.

The backward pass runs the mirrored pipeline (combine-backward is dispatch shaped and also
produces the gate gradients; dispatch-backward is combine shaped).  Both paths place rows at
positions the ORIGIN computes from the all-gathered expert histogram, so the expert GEMMs see
identical inputs and the two paths agree bit for bit.

Reference counterparts: ``terrace/ep_dist.py:82-122`` and ``terrace/ta2a_fwd.py:445-670`` (which
issue 4 and 9 collectives with 1-3 host syncs per forward).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..routing import TRouteConfig
from ..utils import trace
from ..utils.flags import flag_bool, flag_int

# arena sections (must match section_offset() in symm_bindings.cpp)
XIN, YOUT, DOUT, DXS, HA_ROWS, RED, HB_ROWS, DRED = range(8)
# flag kinds (must match Tb200FlagKind)
(FK_COUNTS, FK_HOPA, FK_DATA, FK_OUT, FK_RED, FK_B_HOPA, FK_B_DATA, FK_B_DG, FK_B_OUT,
 FK_B_RED) = range(10)
FK_NUM = 10
MAX_WORLD = 16
SEG_ALIGN = 64          # expert segments start on multiples of 64 rows (zero padding rows)

LIVE = {"one_hop_fwd": 0, "two_hop_fwd": 0, "one_hop_bwd": 0, "two_hop_bwd": 0, "echo": 0,
        "epilogue_push_fwd": 0, "epilogue_push_bwd": 0, "push_back": 0}


def _lib():
    from ..ops.native import _lib as counted
    return counted()


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


GUARD_BYTES = 256       # canary words after every arena section
GUARD_VALUE = 0xA5


def arena_layout(sizes, guard: int = GUARD_BYTES):
    """Offsets of the arena's sections, each followed by ``guard`` canary bytes that no kernel
    may touch: ``(offsets, guard_offsets, total_bytes)``.  Sections start 256-byte aligned."""
    offsets, guards, off = [], [], 0
    for s in sizes:
        offsets.append(off)
        off += _align(s)
        guards.append(off)
        off += _align(guard) if guard > 0 else 0
    return offsets, guards, off


class FusedEPContext:
    def __init__(self, cfg: TRouteConfig, hidden: int, d_expert: int, tokens: int, *, world: int,
                 rank: int, rpn: int, device, group=None, row_capacity_factor: float = 2.0,
                 epilogue_push=None):
        from .. import ops
        if not ops.custom_ops_enabled():
            raise RuntimeError("the fused transport needs the native library: "
                               + ops.status().reason)
        self._init_args = dict(cfg=cfg, hidden=hidden, d_expert=d_expert, tokens=tokens,
                               world=world, rank=rank, rpn=rpn, device=device, group=group,
                               row_capacity_factor=row_capacity_factor,
                               epilogue_push=epilogue_push)
        if world > MAX_WORLD:
            raise ValueError(f"world={world} exceeds the arena limit {MAX_WORLD}")
        if cfg.n_experts % world or world % rpn:
            raise ValueError("n_experts % world and world % rpn must be zero")
        self.cfg, self.hidden, self.d_expert, self.tokens = cfg, hidden, d_expert, tokens
        self.world, self.rank, self.rpn, self.device = world, rank, rpn, torch.device(device)
        self.group = group
        self.E = cfg.n_experts
        self.epr = self.E // world
        self.n_nodes = world // rpn
        self.k, self.M, self.q = cfg.top_k, cfg.top_groups, cfg.per_group_k
        self.two_hop_ok = (self.n_nodes >= 2 and cfg.n_groups == self.n_nodes)
        self.cap_rows = _align(min(world * tokens * self.k,
                                   int(row_capacity_factor * tokens * self.k))
                               + self.epr * (SEG_ALIGN - 1), 128)
        self.epoch = 0
        if epilogue_push is None:
            epilogue_push = flag_bool("TERRACE_EP_EPILOGUE_PUSH")
        self.epilogue_push = bool(epilogue_push)
        # two-hop return leg: the representative stores its reduced rows into the origin's section
        # instead of the origin reading them remotely (off by default; not yet run on a GPU)
        self.push_back = flag_bool("TERRACE_EP_PUSH_BACK")
        self.ret_slots = tokens * self.k
        H = hidden
        sizes = [
            world * self.E * 4,                      # counts_all
            FK_NUM * MAX_WORLD * 4,                  # flags
            self.cap_rows * H * 2,                   # xin
            self.cap_rows * H * 2,                   # yout
            self.cap_rows * H * 2,                   # dout
            self.cap_rows * H * 2,                   # dxs
        ]
        arows = self.n_nodes * tokens if self.two_hop_ok else 1
        sizes += [arows * H * 2, arows * 3 * self.q * 4, arows * H * 2, arows * H * 2,
                  arows * H * 2, arows * self.q * 4]
        if self.epilogue_push:      # return slots (forward, backward) and the owners' row map
            sizes += [self.ret_slots * H * 2, self.ret_slots * H * 2, self.cap_rows * 4]
        self.offsets, self.guards, self.nbytes = arena_layout(sizes)
        lib = torch.ops.terrace
        dev_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.buf = lib.symm_alloc(self.nbytes, dev_index)
        self._guard_index = (torch.tensor(self.guards, dtype=torch.int64, device=self.device)
                             .unsqueeze(1) + torch.arange(GUARD_BYTES, device=self.device))
        self.buf[self._guard_index.reshape(-1)] = GUARD_VALUE
        handle = lib.symm_ipc_handle(self.buf)
        handles = [None] * world
        dist.all_gather_object(handles, handle.numpy().tobytes(), group=group)
        self.peer_ptrs = []
        self._opened = []
        for r in range(world):
            if r == rank:
                self.peer_ptrs.append(self.buf.data_ptr())
            else:
                h = torch.frombuffer(bytearray(handles[r]), dtype=torch.uint8)
                p = lib.symm_ipc_open(h, dev_index)
                self._opened.append(p)
                self.peer_ptrs.append(p)
        geom = [world, rank, self.E, self.epr, rpn, self.n_nodes, tokens, self.k, self.M, self.q,
                H, self.cap_rows]
        self.arena = lib.symm_make_arena(self.peer_ptrs, self.offsets[:12], geom)
        if self.epilogue_push:
            self.off_ret, self.off_dret, self.off_rowmap = self.offsets[12:15]
            self.ret_base = torch.tensor([p + self.off_ret for p in self.peer_ptrs],
                                         dtype=torch.int64, device=self.device)
            self.dret_base = torch.tensor([p + self.off_dret for p in self.peer_ptrs],
                                          dtype=torch.int64, device=self.device)
            self.row_map = self.buf[self.off_rowmap: self.off_rowmap + self.cap_rows * 4].view(
                torch.int32)
        self.done = torch.zeros(8, dtype=torch.int32, device=self.device)
        self._dev_index = dev_index
        dist.barrier(group=group)

    # views of this rank's own sections
    def section(self, sel: int) -> torch.Tensor:
        off = self.offsets[2 + sel] if sel < 4 else self.offsets[{4: 6, 5: 8, 6: 9, 7: 10}[sel]]
        rows = self.cap_rows if sel < 4 else self.n_nodes * self.tokens
        n = rows * self.hidden * 2
        return self.buf[off: off + n].view(torch.bfloat16).view(rows, self.hidden)

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def owner_wait_range(self, mode: str):
        """Which arrival flags an expert owner waits for: every rank (one-hop) or the ranks of
        its own group (two-hop, where the group's representatives forward the rows)."""
        if mode == "one_hop":
            return 0, self.world
        return (self.rank // self.rpn) * self.rpn, self.rpn

    def close(self):
        lib = torch.ops.terrace
        for p in self._opened:
            lib.symm_ipc_close(p, self._dev_index)
        self._opened = []

    def rebuild(self) -> None:
        """Recovery after a reported failure (a wait that ran out, a bad index): every rank of
        the group calls this between steps.  The peers' mappings are closed, then (after a
        barrier, so that nobody frees memory a peer still maps) the arena is freed and a fresh one
        with the same geometry is allocated, exchanged and mapped; epochs restart at zero."""
        args = self._init_args
        torch.cuda.synchronize(self.device)
        self.close()
        if self.world > 1:
            dist.barrier(group=self.group)
        self.buf = self.arena = self.peer_ptrs = self.row_map = None   # views keep the storage alive
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)
        self.take_status()
        self.__init__(args["cfg"], args["hidden"], args["d_expert"], args["tokens"],
                      world=args["world"], rank=args["rank"], rpn=args["rpn"],
                      device=args["device"], group=args["group"],
                      row_capacity_factor=args["row_capacity_factor"],
                      epilogue_push=args["epilogue_push"])

    def take_status(self) -> int:
        return int(torch.ops.terrace.symm_take_status(self._dev_index))

    def check_canaries(self) -> list:
        """Indices of the arena sections whose trailing canary bytes were overwritten (by this
        rank's kernels or by a peer's stores).  One host synchronisation; for tests and for
        debugging, not for the step."""
        bad = (self.buf[self._guard_index.reshape(-1)].view(len(self.guards), GUARD_BYTES)
               != GUARD_VALUE).any(dim=1)
        return torch.nonzero(bad).flatten().tolist()


def _plan(ctx: FusedEPContext, idx, gates, mode: str, ep: int):
    lib = _lib()
    es, gs, cols, rank_local, chunk_hist = lib.ep_plan_pass1(
        idx.contiguous(), gates.detach().float().contiguous(), ctx.E)
    ranka = chunka = None
    if mode == "two_hop":
        ranka, chunka = lib.hopa_rank(ctx.arena, es)
    my_base, seg_start, seg_count, rows_a = lib.ep_plan(ctx.arena, chunk_hist, chunka, ep,
                                                        SEG_ALIGN)
    return dict(es=es, gs=gs, cols=cols, rank_local=rank_local, chunk_hist=chunk_hist,
                ranka=ranka, chunka=chunka, my_base=my_base, seg_start=seg_start,
                seg_count=seg_count, rows_a=rows_a)


def _dispatch(ctx, p, x, mode: str, ep: int):
    """Forward dispatch: rows of ``x`` land in the owners' ``xin`` sections."""
    lib = _lib()
    if mode == "one_hop" and ctx.epilogue_push:
        pos, _ = lib.ep_push_ret(ctx.arena, x, p["es"], p["rank_local"], p["chunk_hist"],
                                 p["my_base"], None, False, XIN, 0, False, FK_DATA, ep,
                                 ctx.done[0:1], ctx.off_rowmap, ctx.ret_slots)
        p["pos"], p["rowa"] = pos, None
    elif mode == "one_hop":
        pos, _ = lib.ep_push(ctx.arena, x, p["es"], p["rank_local"], p["chunk_hist"],
                             p["my_base"], None, False, XIN, XIN, FK_DATA, ep, ctx.done[0:1])
        p["pos"], p["rowa"] = pos, None
    else:
        pos, rowa = lib.hopa_push(ctx.arena, x, p["es"], p["gs"], p["rank_local"],
                                  p["chunk_hist"], p["my_base"], p["ranka"], p["chunka"], None,
                                  HA_ROWS, True, FK_HOPA, ep, ctx.done[0:1])
        lib.arrival_push(ctx.arena, p["rows_a"], HA_ROWS, XIN, XIN, False, False, FK_HOPA,
                         FK_DATA, -1, ep, ctx.done[1:2])
        p["pos"], p["rowa"] = pos, rowa


def _signal_out(ctx, mode: str, kind: int, ep: int, like, wait_kind: int = -1):
    lib = _lib()
    first, n = ctx.owner_wait_range(mode)
    lib.ep_signal(ctx.arena, kind, first, n, 1, ctx.rank, ep, wait_kind, first, n, like)


def _combine(ctx, p, mode: str, ep: int, *, src: int, use_gate: bool, backward: bool,
             pull: bool = False):
    """``pull`` forces the remote-read combine even on a context with ``epilogue_push`` (the
    echo measurement has no GEMM whose epilogue could have delivered the rows)."""
    lib = _lib()
    out_kind = FK_B_OUT if backward else FK_OUT
    if mode == "one_hop" and ctx.epilogue_push and not pull:
        return lib.ep_combine_local(ctx.arena, p["pos"], p["es"], p["gs"] if use_gate else None,
                                    ctx.off_dret if backward else ctx.off_ret, ctx.ret_slots,
                                    ctx.cfg.group_size, out_kind, ep)
    if mode == "one_hop":
        return lib.ep_pull_combine(ctx.arena, p["pos"], p["es"], p["gs"] if use_gate else None,
                                   src, ctx.cfg.group_size, out_kind, ep)
    red_sel, red_kind = (DRED, FK_B_RED) if backward else (RED, FK_RED)
    push = bool(getattr(ctx, "push_back", False))
    lib.arrival_combine(ctx.arena, p["rows_a"], src, red_sel, use_gate, out_kind, red_kind, ep,
                        ctx.done[2:3], push)
    if push:
        LIVE["push_back"] += 1
    return lib.origin_combine(ctx.arena, p["es"], p["rowa"], red_sel, red_kind, ep, push)


class _FusedMoE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gates, w13, w2, idx, fctx: FusedEPContext, mode: str):
        lib = _lib()
        ep = fctx.next_epoch()
        xc = x.contiguous()
        with trace.phase("ep.fwd.plan"):
            p = _plan(fctx, idx, gates, mode, ep)
        with trace.phase("ep.fwd.dispatch"):
            _dispatch(fctx, p, xc, mode, ep)
        first, n = fctx.owner_wait_range(mode)
        d = w2.shape[1]
        xin, yout = fctx.section(XIN), fctx.section(YOUT)
        act = torch.empty(fctx.cap_rows, d, dtype=torch.bfloat16, device=x.device)
        need = any(ctx.needs_input_grad)
        h13 = (torch.empty(fctx.cap_rows, 2 * d, dtype=torch.bfloat16, device=x.device)
               if need else None)
        scatter = mode == "one_hop" and fctx.epilogue_push
        with trace.phase("ep.fwd.experts"):
            if need:      # the weight gradient reads the padding rows of xin: keep them zero
                lib.zero_pad_rows(xin, p["seg_start"], p["seg_count"], SEG_ALIGN)
            lib.grouped_gemm_ex(xin, w13.contiguous(), act, h13, p["seg_start"], p["seg_count"],
                                0, 1, fctx.arena, FK_DATA, first, n, ep, SEG_ALIGN)
            if scatter:     # GEMM 2 stores every output row into its origin's return slot
                lib.grouped_gemm_scatter(act, w2.contiguous(), p["seg_start"], p["seg_count"], 0,
                                         fctx.row_map, fctx.ret_base, fctx.ret_slots)
                LIVE["epilogue_push_fwd"] += 1
            else:
                lib.grouped_gemm_ex(act, w2.contiguous(), yout, None, p["seg_start"],
                                    p["seg_count"], 0, 0, None, 0, 0, 0, ep, SEG_ALIGN)
        with trace.phase("ep.fwd.combine"):
            _signal_out(fctx, mode, FK_OUT, ep, xc)
            y = _combine(fctx, p, mode, ep, src=YOUT, use_gate=True, backward=False)
        ctx.fctx, ctx.mode, ctx.ep, ctx.plan = fctx, mode, ep, p
        ctx.save_for_backward(w13, w2, act, h13 if h13 is not None else act)
        ctx.gate_dtype = gates.dtype
        LIVE[f"{mode}_fwd"] += 1
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib()
        fctx, mode, ep, p = ctx.fctx, ctx.mode, ctx.ep, ctx.plan
        w13, w2, act, h13 = ctx.saved_tensors
        dyc = dy.contiguous()
        first, n = fctx.owner_wait_range(mode)
        scatter = mode == "one_hop" and fctx.epilogue_push
        tr_dispatch = trace.phase("ep.bwd.dispatch")
        tr_dispatch.__enter__()
        if scatter:     # the saved expert outputs sit in my own return slots
            _, dgs = lib.ep_push_ret(fctx.arena, dyc, p["es"], p["rank_local"], p["chunk_hist"],
                                     p["my_base"], p["gs"], True, DOUT, fctx.off_ret, True,
                                     FK_B_DATA, ep, fctx.done[0:1], fctx.off_rowmap,
                                     fctx.ret_slots)
        elif mode == "one_hop":
            _, dgs = lib.ep_push(fctx.arena, dyc, p["es"], p["rank_local"], p["chunk_hist"],
                                 p["my_base"], p["gs"], True, DOUT, YOUT, FK_B_DATA, ep,
                                 fctx.done[0:1])
        else:
            lib.hopa_push(fctx.arena, dyc, p["es"], p["gs"], p["rank_local"], p["chunk_hist"],
                          p["my_base"], p["ranka"], p["chunka"], p["rowa"], HB_ROWS, False,
                          FK_B_HOPA, ep, fctx.done[0:1])
            lib.arrival_push(fctx.arena, p["rows_a"], HB_ROWS, DOUT, YOUT, True, True, FK_B_HOPA,
                             FK_B_DATA, FK_B_DG, ep, fctx.done[1:2])
        tr_dispatch.__exit__(None, None, None)
        xin, dout, dxs = fctx.section(XIN), fctx.section(DOUT), fctx.section(DXS)
        d = w2.shape[1]
        dact = torch.empty(fctx.cap_rows, d, dtype=torch.bfloat16, device=dy.device)
        tr_experts = trace.phase("ep.bwd.experts")
        tr_experts.__enter__()
        lib.zero_pad_rows(dout, p["seg_start"], p["seg_count"], SEG_ALIGN)
        lib.grouped_gemm_ex(dout, w2.contiguous(), dact, None, p["seg_start"], p["seg_count"], 1,
                            0, fctx.arena, FK_B_DATA, first, n, ep, SEG_ALIGN)
        dw2 = lib.grouped_wgrad(act, dout, p["seg_start"], p["seg_count"], 0, SEG_ALIGN)
        dh13 = lib.swiglu_bwd(h13, dact)
        dw13 = lib.grouped_wgrad(xin, dh13, p["seg_start"], p["seg_count"], 0, SEG_ALIGN)
        if scatter:
            lib.grouped_gemm_scatter(dh13, w13.contiguous(), p["seg_start"], p["seg_count"], 1,
                                     fctx.row_map, fctx.dret_base, fctx.ret_slots)
            LIVE["epilogue_push_bwd"] += 1
        else:
            lib.grouped_gemm_ex(dh13, w13.contiguous(), dxs, None, p["seg_start"],
                                p["seg_count"], 1, 0, None, 0, 0, 0, ep, SEG_ALIGN)
        tr_experts.__exit__(None, None, None)
        with trace.phase("ep.bwd.combine"):
            _signal_out(fctx, mode, FK_B_OUT, ep, dyc)
            dx = _combine(fctx, p, mode, ep, src=DXS, use_gate=False, backward=True)
            if mode == "two_hop":
                dgs = lib.origin_pull_dgate(fctx.arena, p["es"], p["rowa"], FK_B_DG, ep)
        dgates = torch.zeros_like(dgs).scatter_(1, p["cols"].long(), dgs).to(ctx.gate_dtype)
        LIVE[f"{mode}_bwd"] += 1
        return dx, dgates, dw13, dw2, None, None, None


def fused_moe_forward(fctx: FusedEPContext, x, idx, gates, w13, w2, *, mode: str):
    """Routed-expert output for this rank's tokens over the fused transport."""
    if mode == "two_hop" and not fctx.two_hop_ok:
        mode = "one_hop"          # fewer than two groups (or groups != routing groups)
    if x.shape[0] > fctx.tokens:
        raise ValueError(f"{x.shape[0]} tokens exceed the context capacity {fctx.tokens}")
    if x.dtype != torch.bfloat16 or w13.dtype != torch.bfloat16:
        raise TypeError("the fused transport moves bf16 rows")
    return _FusedMoE.apply(x, gates, w13, w2, idx, fctx, mode)


def pipeline_depth() -> int:
    """``TERRACE_EP_PIPELINE=n`` (default 1 = off): run the fused layer on ``n`` token slices."""
    return flag_int("TERRACE_EP_PIPELINE", 1, 1, 8)


class PipelinedFusedEP:
    """Token-sliced software pipeline over the fused transport: ``n`` independent arenas, each
    slice of the tokens runs plan -> push -> GEMMs -> combine on its own CUDA stream, so that the
    dispatch and combine of one slice overlap the expert GEMMs of another.  The kernels are the
    unchanged ones of the unsliced path.

    Why this cannot deadlock although the GEMM kernels spin on flags: a slice's kernels wait only
    for the SAME slice's pushes of OTHER GPUs; its own push precedes them in stream order; pushes
    never wait; and slices never wait for each other.  Every chain of waits therefore ends in a
    push kernel, which needs no shared memory and is always schedulable beside a resident GEMM.
    If the hardware does not co-schedule the streams, the slices simply run one after another.

    Numerics: every token's output and input gradient equal the unsliced path bit for bit (a
    row's products do not depend on which tile it sits in); weight gradients are the sum of the
    slices' partial gradients, so they differ from the unsliced ones by rounding.  One-hop and
    two-hop still agree bit for bit under the same slicing."""

    def __init__(self, cfg: TRouteConfig, hidden: int, d_expert: int, tokens: int, *, n: int,
                 world: int, rank: int, rpn: int, device, group=None, **kw):
        if n < 2:
            raise ValueError("a pipeline needs at least two slices")
        self.n, self.tokens = n, tokens
        self.slice_tokens = (tokens + n - 1) // n
        self.ctxs = [FusedEPContext(cfg, hidden, d_expert, self.slice_tokens, world=world,
                                    rank=rank, rpn=rpn, device=device, group=group, **kw)
                     for _ in range(n)]
        self.device = torch.device(device)
        self.streams = ([torch.cuda.Stream(device=self.device) for _ in range(n)]
                        if self.device.type == "cuda" else [None] * n)
        self.two_hop_ok = self.ctxs[0].two_hop_ok
        self.cfg = cfg

    def bounds(self, T: int):
        step = (T + self.n - 1) // self.n
        return [(lo, min(T, lo + step)) for lo in range(0, T, step)]

    def forward(self, x, idx, gates, w13, w2, *, mode: str):
        if x.shape[0] > self.tokens:
            raise ValueError(f"{x.shape[0]} tokens exceed the context capacity {self.tokens}")
        outs = []
        cur = torch.cuda.current_stream(self.device) if self.streams[0] is not None else None
        for (lo, hi), ctx, st in zip(self.bounds(x.shape[0]), self.ctxs, self.streams):
            if st is None:
                outs.append(fused_moe_forward(ctx, x[lo:hi], idx[lo:hi], gates[lo:hi], w13, w2,
                                              mode=mode))
                continue
            st.wait_stream(cur)
            with torch.cuda.stream(st):
                y = fused_moe_forward(ctx, x[lo:hi], idx[lo:hi], gates[lo:hi], w13, w2, mode=mode)
            for t in (x, idx, gates, w13, w2):      # allocated on the caller's stream, read on st
                t.record_stream(st)
            y.record_stream(cur)                    # allocated on st, read on the caller's stream
            outs.append(y)
        if cur is not None:
            for st in self.streams[:len(outs)]:
                cur.wait_stream(st)
        return torch.cat(outs, dim=0)

    def take_status(self) -> int:
        return max(c.take_status() for c in self.ctxs)

    def check_canaries(self) -> list:
        return [(i, sec) for i, c in enumerate(self.ctxs) for sec in c.check_canaries()]

    def close(self) -> None:
        for c in self.ctxs:
            c.close()

    def rebuild(self) -> None:
        for c in self.ctxs:
            c.rebuild()


def make_context(cfg: TRouteConfig, hidden: int, d_expert: int, tokens: int, **kw):
    """A ``FusedEPContext``, or a ``PipelinedFusedEP`` when ``TERRACE_EP_PIPELINE`` asks for one."""
    n = pipeline_depth()
    if n > 1 and kw.get("world", 1) > 1:
        return PipelinedFusedEP(cfg, hidden, d_expert, tokens, n=n, **kw)
    return FusedEPContext(cfg, hidden, d_expert, tokens, **kw)


def run_fused(ctx, x, idx, gates, w13, w2, *, mode: str):
    if isinstance(ctx, PipelinedFusedEP):
        return ctx.forward(x, idx, gates, w13, w2, mode=mode)
    return fused_moe_forward(ctx, x, idx, gates, w13, w2, mode=mode)


@torch.no_grad()
def fused_dispatch_combine(fctx: FusedEPContext, x, idx, gates, *, mode: str):
    """Dispatch immediately followed by combine (rows echo back unchanged, gate-weighted): the
    communication-only measurement."""
    if isinstance(fctx, PipelinedFusedEP):      # slice after slice on the caller's stream
        return torch.cat([fused_dispatch_combine(c, x[lo:hi], idx[lo:hi], gates[lo:hi], mode=mode)
                          for (lo, hi), c in zip(fctx.bounds(x.shape[0]), fctx.ctxs)], dim=0)
    if mode == "two_hop" and not fctx.two_hop_ok:
        mode = "one_hop"
    ep = fctx.next_epoch()
    p = _plan(fctx, idx, gates, mode, ep)
    _dispatch(fctx, p, x.contiguous(), mode, ep)
    _signal_out(fctx, mode, FK_OUT, ep, x, wait_kind=FK_DATA)
    LIVE["echo"] += 1
    return _combine(fctx, p, mode, ep, src=XIN, use_gate=True, backward=False, pull=True)
