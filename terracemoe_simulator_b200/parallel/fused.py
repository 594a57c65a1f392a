"""Fused expert parallelism over peer memory: the product path for dispatch / combine.

``FusedEPContext`` owns one symmetric arena per MoE layer (see ``ops/csrc/symm_layout.h``): every
rank ``cudaMalloc``s the same layout, exports it with CUDA IPC, and maps all peers.  The kernels
(``ops/csrc/symm.cu``) then move token rows with plain peer stores/loads and synchronise with
epoch flags; NCCL is used only to exchange the IPC handles at start-up.

Default schedule (``overlap``; no host synchronisation anywhere, nothing is read remotely):

  one-hop   plan -> the push of the rows runs on a side stream in ``chunks`` launches, one per
            range of local experts, each raising the owners' arrival flags a little further ->
            per chunk: [GEMM 1 waits for the flag value of its expert range] SwiGLU GEMM, then
            GEMM 2 whose epilogue stores every output row straight into the ORIGIN's return slot
            over NVLink -> signal -> the origin reduces its k slots from local memory
  two-hop   plan -> Hop A push (one row per (token, group) + header) to the representative ->
            the representative forwards every (row, pick) to the owner (Hop B), again chunk by
            chunk on the side stream -> per chunk: gated SwiGLU GEMM, GEMM 2 storing each row
            into the REPRESENTATIVE's return slot -> the representative applies the gates and
            reduces the q picks of a row from local memory and stores the result into the
            origin's section -> the origin adds its M group rows from local memory

  so the transfer of chunk c + 1 runs under the GEMMs of chunk c, the return transfer is part of
  the second GEMM, and the only exposed communication is the first chunk's push and the final
  local reduction.  The backward pass mirrors it (combine-backward is dispatch shaped and also
  produces the gate gradients; dispatch-backward is combine shaped).

Why the side stream cannot deadlock although GEMM kernels spin on flags: a GEMM only waits for
pushes of OTHER GPUs (its own GPU's push of the same chunk precedes it through an event); pushes
wait for nothing but, in the two-hop case, other GPUs' Hop A pushes, which wait for nothing; and
a push kernel needs no shared memory, so it is always schedulable beside a resident GEMM.

``TERRACE_EP_OVERLAP=0`` keeps the earlier schedule as the A/B arm: one push launch, plain GEMMs
into the owner's output section, and a combine that reads the owners' rows remotely.

Both schedules and both hops place rows at positions the ORIGIN computes from the all-gathered
expert histogram and reduce in the same canonical order, so one-hop and two-hop agree bit for
bit with each other and across schedules.

One forward may be outstanding per context: the backward reads the forward's rows from the
arena, so a second forward before the backward of the first would overwrite them.  The context
refuses that with an error instead of returning wrong gradients.

Reference counterparts: ``terrace/ep_dist.py:82-122`` and ``terrace/ta2a_fwd.py:445-670`` (which
issue 4 and 9 collectives with 1-3 host syncs per forward); the overlap window of the seam,
``terrace/ta2a_dispatch.py:765-778``.
"""
from __future__ import annotations

import math
import weakref

import torch
import torch.distributed as dist

from ..routing import TRouteConfig
from ..utils import trace
from ..utils.flags import flag_bool, flag_int

# arena sections with a selector in the native ops (must match section_offset() in
# symm_bindings.cpp)
XIN, YOUT, DOUT, DXS, HA_ROWS, RED, HB_ROWS, DRED = range(8)
# flag kinds (must match Tb200FlagKind)
(FK_COUNTS, FK_HOPA, FK_DATA, FK_OUT, FK_RED, FK_B_HOPA, FK_B_DATA, FK_B_DG, FK_B_OUT,
 FK_B_RED) = range(10)
FK_NUM = 10
MAX_WORLD = 16
SEG_ALIGN = 64          # expert segments start on multiples of 64 rows (zero padding rows)
MAX_CHUNKS = 8
FLAG_STRIDE = 16        # data flags take the values epoch * 16 + (chunks landed), 15 = all

LIVE = {"one_hop_fwd": 0, "two_hop_fwd": 0, "one_hop_bwd": 0, "two_hop_bwd": 0, "echo": 0,
        "overlap_fwd": 0, "overlap_bwd": 0, "chunk_pushes": 0}

# names of the arena sections in layout order; the first twelve fill the native descriptor
_BASE_SECTIONS = ("counts_all", "flags", "xin", "yout", "dout", "dxs", "ha_rows", "ha_hdr", "red",
                  "hb_rows", "dred", "dgate")
_SEL_NAME = {XIN: "xin", YOUT: "yout", DOUT: "dout", DXS: "dxs", HA_ROWS: "ha_rows", RED: "red",
             HB_ROWS: "hb_rows", DRED: "dred"}


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


def section_sizes(*, world: int, n_experts: int, hidden: int, q: int, cap_rows: int,
                  arrival_rows: int, out_rows: int, overlap: bool, own_slots: int,
                  rep_slots: int) -> dict:
    """Bytes of every arena section, in layout order.  ``cap_rows``: rows of the expert-sorted
    buffers; ``arrival_rows``: Hop A rows a representative can receive (1 when two-hop is not
    used); ``out_rows``: rows of the owner-side output sections (1 under the overlap schedule);
    ``own_slots`` / ``rep_slots``: return slots at the origin (one-hop) and at the
    representative (two-hop), 1 for a path the context does not run."""
    row = hidden * 2
    sizes = {
        "counts_all": world * n_experts * 4, "flags": FK_NUM * MAX_WORLD * 4,
        "xin": cap_rows * row, "yout": out_rows * row, "dout": cap_rows * row,
        "dxs": out_rows * row, "ha_rows": arrival_rows * row,
        "ha_hdr": arrival_rows * 3 * q * 4, "red": arrival_rows * row,
        "hb_rows": arrival_rows * row, "dred": arrival_rows * row, "dgate": arrival_rows * q * 4,
    }
    if overlap:
        sizes.update({"ret": own_slots * row, "dret": own_slots * row, "rowmap": cap_rows * 4,
                      "ret2": rep_slots * row, "dret2": rep_slots * row})
    return sizes


def chunk_ranges(epr: int, chunks: int):
    """Split the local experts ``0 .. epr`` into at most ``chunks`` contiguous ranges of (almost)
    equal length: ``[(lo, hi), ...]``."""
    n = max(1, min(int(chunks), epr, MAX_CHUNKS))
    base, extra = divmod(epr, n)
    out, lo = [], 0
    for i in range(n):
        hi = lo + base + (1 if i < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


def flag_value(epoch: int, i: int, n: int) -> int:
    """Value of the data flags once chunk ``i`` of ``n`` has landed (the last one writes 15)."""
    return epoch * FLAG_STRIDE + (FLAG_STRIDE - 1 if i == n - 1 else i + 1)


class FusedEPContext:
    def __init__(self, cfg: TRouteConfig, hidden: int, d_expert: int, tokens: int, *, world: int,
                 rank: int, rpn: int, device, group=None, row_capacity_factor: float = 2.0,
                 overlap=None, chunks=None, modes=None):
        from .. import ops
        if not ops.custom_ops_enabled():
            raise RuntimeError("the fused transport needs the native library: "
                               + ops.status().reason)
        if overlap is None:
            overlap = flag_bool("TERRACE_EP_OVERLAP", True)
        if chunks is None:
            chunks = flag_int("TERRACE_EP_CHUNKS", 2, 1, MAX_CHUNKS)
        self._init_args = dict(cfg=cfg, hidden=hidden, d_expert=d_expert, tokens=tokens,
                               world=world, rank=rank, rpn=rpn, device=device, group=group,
                               row_capacity_factor=row_capacity_factor, overlap=overlap,
                               chunks=chunks, modes=modes)
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
        # ``modes`` names the paths the context will run (default both): the sections only the
        # other path uses shrink to one row, which is most of the arena at training sizes
        modes = ("one_hop", "two_hop") if modes is None else tuple(modes)
        if not modes or any(m not in ("one_hop", "two_hop") for m in modes):
            raise ValueError(f"modes must name one_hop and / or two_hop, got {modes!r}")
        self.two_hop_ok = (self.n_nodes >= 2 and cfg.n_groups == self.n_nodes
                           and "two_hop" in modes)
        # a two-hop request on a geometry without two groups runs one-hop: keep its sections
        self.one_hop_ok = "one_hop" in modes or not self.two_hop_ok
        self.cap_rows = _align(min(world * tokens * self.k,
                                   int(row_capacity_factor * tokens * self.k))
                               + self.epr * (SEG_ALIGN - 1), 128)
        self.epoch = 0
        self.overlap = bool(overlap)
        self.chunks = chunk_ranges(self.epr, chunks if self.overlap else 1)
        self.ret_slots = tokens * self.k
        H = hidden
        arows = self.n_nodes * tokens if self.two_hop_ok else 1
        self.arows = arows
        self.ret2_slots = arows * self.q
        # with the overlap schedule the second GEMM stores into return slots, so the owner-side
        # output sections are never touched
        out_rows = 1 if self.overlap else self.cap_rows
        sizes = section_sizes(world=world, n_experts=self.E, hidden=H, q=self.q,
                              cap_rows=self.cap_rows, arrival_rows=arows, out_rows=out_rows,
                              overlap=self.overlap,
                              own_slots=self.ret_slots if self.one_hop_ok else 1,
                              rep_slots=self.ret2_slots if self.two_hop_ok else 1)
        names = list(sizes)
        assert tuple(names[:12]) == _BASE_SECTIONS
        offsets, self.guards, self.nbytes = arena_layout([sizes[n] for n in names])
        self.off = dict(zip(names, offsets))
        self.offsets = offsets
        self._rows = {"xin": self.cap_rows, "yout": out_rows, "dout": self.cap_rows,
                      "dxs": out_rows, "ha_rows": arows, "red": arows, "hb_rows": arows,
                      "dred": arows}
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
        self.arena = lib.symm_make_arena(self.peer_ptrs, offsets[:12], geom)
        self.row_map = None
        if self.overlap:
            def bases(name):
                return torch.tensor([p + self.off[name] for p in self.peer_ptrs],
                                    dtype=torch.int64, device=self.device)
            self.ret_base, self.dret_base = bases("ret"), bases("dret")
            self.ret2_base, self.dret2_base = bases("ret2"), bases("dret2")
            o = self.off["rowmap"]
            self.row_map = self.buf[o: o + self.cap_rows * 4].view(torch.int32)
        self.done = torch.zeros(8, dtype=torch.int32, device=self.device)
        self._dev_index = dev_index
        self.side = torch.cuda.Stream(device=self.device) if self.overlap else None
        self._events = [torch.cuda.Event() for _ in range(MAX_CHUNKS)] if self.overlap else []
        self._inflight = None       # weak reference to the autograd context of a forward whose
        #                             backward has not run yet
        dist.barrier(group=group)

    # views of this rank's own sections
    def section(self, sel: int) -> torch.Tensor:
        name = _SEL_NAME[sel]
        rows = self._rows[name]
        off = self.off[name]
        n = rows * self.hidden * 2
        return self.buf[off: off + n].view(torch.bfloat16).view(rows, self.hidden)

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def mark_link_quiet(self) -> None:
        """Called by the backward pass where the longest stretch without NVLink traffic begins
        (the last dispatched gradient rows have arrived; the weight-gradient GEMMs follow)."""
        if self.device.type != "cuda":
            return
        if getattr(self, "_quiet", None) is None:
            self._quiet = torch.cuda.Event()
        self._quiet.record(torch.cuda.current_stream(self.device))

    def link_quiet_event(self):
        """CUDA event of the latest ``mark_link_quiet`` (None before the first backward): work on
        other streams that would compete with the peer traffic -- a host-to-device copy of the
        next input, for one -- can wait for it and run under the weight-gradient GEMMs."""
        return getattr(self, "_quiet", None)

    def check_mode(self, mode: str) -> None:
        if mode == "one_hop" and not self.one_hop_ok:
            raise ValueError("this context was built for two_hop only (modes=('two_hop',)): its "
                             "one-hop return sections hold one row")

    def owner_wait_range(self, mode: str):
        """Which arrival flags an expert owner waits for: every rank (one-hop) or the ranks of
        its own group (two-hop, where the group's representatives forward the rows)."""
        if mode == "one_hop":
            return 0, self.world
        return (self.rank // self.rpn) * self.rpn, self.rpn

    # ---- one outstanding forward -----------------------------------------------------------
    def claim(self, actx) -> None:
        """Called by a forward that will be backwarded: refuses when an earlier forward of this
        context still waits for its backward (its rows in the arena would be overwritten)."""
        self.check_free()
        self._inflight = weakref.ref(actx)

    def check_free(self) -> None:
        held = self._inflight() if self._inflight is not None else None
        if held is not None and not getattr(held, "_terrace_done", False):
            raise RuntimeError(
                "this FusedEPContext still holds the rows of a forward whose backward has not "
                "run: one forward may be outstanding per context (use one context per call "
                "site, or run the earlier backward first)")
        self._inflight = None

    def release(self, actx) -> None:
        actx._terrace_done = True
        if self._inflight is not None and self._inflight() is actx:
            self._inflight = None

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
                      overlap=args["overlap"], chunks=len(self.chunks))

    def take_status(self) -> int:
        return int(torch.ops.terrace.symm_take_status(self._dev_index))

    def status_tensor(self) -> torch.Tensor:
        """The device status word (int32 [1]) without a synchronisation: non-zero once a kernel of
        this device skipped a row (arena overflow), gave up a wait, ...  For a deferred read."""
        return torch.ops.terrace.symm_status_tensor(self._dev_index)

    def check_canaries(self) -> list:
        """Indices of the arena sections whose trailing canary bytes were overwritten (by this
        rank's kernels or by a peer's stores).  One host synchronisation; for tests and for
        debugging, not for the step."""
        bad = (self.buf[self._guard_index.reshape(-1)].view(len(self.guards), GUARD_BYTES)
               != GUARD_VALUE).any(dim=1)
        return torch.nonzero(bad).flatten().tolist()


def expert_capacity(capacity_factor, tokens_global: int, top_k: int, n_experts: int) -> int:
    """Rows an expert accepts under ``capacity_factor`` (0 = unbounded); the formula of
    ``layer.apply_capacity``."""
    if capacity_factor is None:
        return 0
    return int(math.ceil(capacity_factor * tokens_global * top_k / n_experts))


def _plan(ctx: FusedEPContext, idx, gates, mode: str, ep: int, cap: int = 0):
    """``cap`` > 0: every expert accepts at most ``cap`` rows in canonical order (source rank,
    then token); the picks beyond it get position -1, are not sent and contribute nothing."""
    lib = _lib()
    es, gs, cols, rank_local, chunk_hist = lib.ep_plan_pass1(
        idx.contiguous(), gates.detach().float().contiguous(), ctx.E)
    ranka = chunka = None
    if mode == "two_hop":
        ranka, chunka = lib.hopa_rank(ctx.arena, es)
    my_base, seg_start, seg_count, rows_a, my_prefix = lib.ep_plan(
        ctx.arena, chunk_hist, chunka, ep, SEG_ALIGN, int(cap))
    return dict(es=es, gs=gs, cols=cols, rank_local=rank_local, chunk_hist=chunk_hist,
                ranka=ranka, chunka=chunka, my_base=my_base, seg_start=seg_start,
                seg_count=seg_count, rows_a=rows_a, my_prefix=my_prefix, cap=int(cap))


def _push_launches(ctx, chunked: bool):
    """``[(i, n, lo, hi)]``: the push launches of one dispatch."""
    ranges = ctx.chunks if chunked else [(0, ctx.epr)]
    return [(i, len(ranges), lo, hi) for i, (lo, hi) in enumerate(ranges)]


def _dispatch(ctx, p, x, mode: str, ep: int, *, backward: bool = False, chunked: bool = False,
              events=None):
    """Dispatch of ``x`` (forward: token rows into the owners' ``xin``; backward: gate-scaled
    gradient rows into the owners' ``dout`` plus the gate gradients) on the current stream.
    With ``chunked`` it is issued as one launch per range of local experts, and ``events[i]`` is
    recorded after launch ``i``.  Returns the gate gradients (backward, one-hop) or None."""
    lib = _lib()
    ov = ctx.overlap
    T = x.shape[0]
    data_kind = FK_B_DATA if backward else FK_DATA
    dst_off = ctx.off["dout" if backward else "xin"]
    launches = _push_launches(ctx, chunked)
    dgs = None

    def mark(i):
        if events:
            events[i].record(torch.cuda.current_stream(ctx.device))
        LIVE["chunk_pushes"] += 1

    if mode == "one_hop":
        if backward:
            pos = p["pos"]
            dgs = torch.empty(T, ctx.k, dtype=torch.float32, device=x.device)
            dot_off = ctx.off["ret"] if ov else ctx.off["yout"]
        else:
            pos = torch.empty(T, ctx.k, dtype=torch.int32, device=x.device)
            dot_off = 0
        for i, n, lo, hi in launches:
            lib.ep_push(ctx.arena, x, p["es"], p["rank_local"], p["chunk_hist"], p["my_base"],
                        p["gs"] if backward else None, pos, dgs, dst_off, dot_off, ov and backward,
                        data_kind, flag_value(ep, i, n), lo, hi, ctx.done[0:1],
                        ctx.off["rowmap"] if (ov and not backward) else -1, ctx.ret_slots,
                        p["my_prefix"], p["cap"])
            mark(i)
        if not backward:
            p["pos"], p["rowa"] = pos, None
        return dgs
    # two-hop: Hop A in one launch, Hop B forwarded by the representative chunk by chunk
    if backward:
        lib.hopa_push(ctx.arena, x, p["es"], p["gs"], p["rank_local"], p["chunk_hist"],
                      p["my_base"], p["ranka"], p["chunka"], p["rowa"], HB_ROWS, False,
                      FK_B_HOPA, ep, ctx.done[0:1])
    else:
        pos, rowa = lib.hopa_push(ctx.arena, x, p["es"], p["gs"], p["rank_local"],
                                  p["chunk_hist"], p["my_base"], p["ranka"], p["chunka"], None,
                                  HA_ROWS, True, FK_HOPA, ep, ctx.done[0:1], p["my_prefix"],
                                  p["cap"])
        p["pos"], p["rowa"] = pos, rowa
    for i, n, lo, hi in launches:
        last = i == n - 1
        if backward:
            lib.arrival_push(ctx.arena, p["rows_a"], HB_ROWS, dst_off,
                             ctx.off["ret2"] if ov else ctx.off["yout"], ov, True, True,
                             FK_B_HOPA, data_kind, FK_B_DG if last else -1, ep,
                             flag_value(ep, i, n), lo, hi, ctx.done[1:2], -1)
        else:
            lib.arrival_push(ctx.arena, p["rows_a"], HA_ROWS, dst_off, 0, False, False, False,
                             FK_HOPA, data_kind, -1, ep, flag_value(ep, i, n), lo, hi,
                             ctx.done[1:2], ctx.off["rowmap"] if ov else -1)
        mark(i)
    return None


def _dispatch_side(ctx, p, x, mode: str, ep: int, *, backward: bool):
    """The chunked dispatch on the context's side stream; returns ``(dgs, events)``.  The caller
    makes the current stream wait for ``events[i]`` before it launches the GEMM of chunk ``i``.
    A context without a side stream issues the same launches in line (``events`` is None)."""
    if ctx.side is None:
        return _dispatch(ctx, p, x, mode, ep, backward=backward, chunked=True), None
    cur = torch.cuda.current_stream(ctx.device)
    ctx.side.wait_stream(cur)
    with torch.cuda.stream(ctx.side):
        dgs = _dispatch(ctx, p, x, mode, ep, backward=backward, chunked=True, events=ctx._events)
    # tensors allocated while the side stream was current are consumed on the caller's stream
    for t in (dgs, p.get("pos"), p.get("rowa")):
        if t is not None:
            t.record_stream(cur)
    return dgs, ctx._events


def _signal_out(ctx, mode: str, kind: int, ep: int, like, wait_kind: int = -1):
    lib = _lib()
    first, n = ctx.owner_wait_range(mode)
    lib.ep_signal(ctx.arena, kind, first, n, 1, ctx.rank, ep, wait_kind, first, n,
                  flag_value(ep, 0, 1), like)


def _combine(ctx, p, mode: str, ep: int, *, src: int, use_gate: bool, backward: bool,
             pull: bool = False):
    """``pull`` forces the remote-read combine even on an overlap context (the echo measurement
    has no GEMM whose epilogue could have delivered the rows)."""
    lib = _lib()
    out_kind = FK_B_OUT if backward else FK_OUT
    local = ctx.overlap and not pull
    if mode == "one_hop":
        if local:
            return lib.ep_pull_combine(ctx.arena, p["pos"], p["es"], p["gs"] if use_gate else None,
                                       ctx.off["dret" if backward else "ret"], ctx.cfg.group_size,
                                       out_kind, ep, ctx.ret_slots)
        return lib.ep_pull_combine(ctx.arena, p["pos"], p["es"], p["gs"] if use_gate else None,
                                   ctx.off[_SEL_NAME[src]], ctx.cfg.group_size, out_kind, ep, 0)
    red_sel, red_kind = (DRED, FK_B_RED) if backward else (RED, FK_RED)
    src_off = ctx.off["dret2" if backward else "ret2"] if local else ctx.off[_SEL_NAME[src]]
    lib.arrival_combine(ctx.arena, p["rows_a"], src_off, red_sel, use_gate, out_kind, red_kind, ep,
                        ctx.done[2:3], local, local)
    return lib.origin_combine(ctx.arena, p["es"], p["rowa"], red_sel, red_kind, ep, local)


class _FusedMoE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gates, w13, w2, idx, fctx: FusedEPContext, mode: str, cap: int = 0):
        lib = _lib()
        need = any(ctx.needs_input_grad)
        if need:
            fctx.claim(ctx)
        else:
            fctx.check_free()
        ep = fctx.next_epoch()
        xc = x.contiguous()
        ov = fctx.overlap
        with trace.phase("ep.fwd.plan"):
            p = _plan(fctx, idx, gates, mode, ep, cap)
        with trace.phase("ep.fwd.dispatch"):
            if ov:
                _, events = _dispatch_side(fctx, p, xc, mode, ep, backward=False)
            else:
                _dispatch(fctx, p, xc, mode, ep)
        first, n = fctx.owner_wait_range(mode)
        d = w2.shape[1]
        xin = fctx.section(XIN)
        act = torch.empty(fctx.cap_rows, d, dtype=torch.bfloat16, device=x.device)
        h13 = (torch.empty(fctx.cap_rows, 2 * d, dtype=torch.bfloat16, device=x.device)
               if need else None)
        w13c, w2c = w13.contiguous(), w2.contiguous()
        ss, sc = p["seg_start"], p["seg_count"]
        with trace.phase("ep.fwd.experts"):
            if need:      # the weight gradient reads the padding rows of xin: keep them zero
                lib.zero_pad_rows(xin, ss, sc, SEG_ALIGN)
            if ov:
                cur = torch.cuda.current_stream(fctx.device) if events else None
                base, slots = ((fctx.ret_base, fctx.ret_slots) if mode == "one_hop"
                               else (fctx.ret2_base, fctx.ret2_slots))
                nch = len(fctx.chunks)
                for i, (lo, hi) in enumerate(fctx.chunks):
                    if cur is not None:
                        cur.wait_event(events[i])
                    lib.grouped_gemm_ex(xin, w13c[lo:hi], act, h13, ss[lo:hi], sc[lo:hi], 0, 1,
                                        fctx.arena, FK_DATA, first, n, flag_value(ep, i, nch),
                                        SEG_ALIGN)
                    # GEMM 2 stores every output row into its return slot (origin / representative)
                    lib.grouped_gemm_scatter(act, w2c[lo:hi], ss[lo:hi], sc[lo:hi], 0,
                                             fctx.row_map, base, slots)
                LIVE["overlap_fwd"] += 1
            else:
                lib.grouped_gemm_ex(xin, w13c, act, h13, ss, sc, 0, 1, fctx.arena, FK_DATA, first,
                                    n, flag_value(ep, 0, 1), SEG_ALIGN)
                lib.grouped_gemm_ex(act, w2c, fctx.section(YOUT), None, ss, sc, 0, 0, None, 0, 0,
                                    0, ep, SEG_ALIGN)
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
        if fctx.epoch != ep:
            raise RuntimeError("the arena of this FusedEPContext was reused by a later forward: "
                               "the rows this backward needs are gone")
        w13, w2, act, h13 = ctx.saved_tensors
        dyc = dy.contiguous()
        first, n = fctx.owner_wait_range(mode)
        ov = fctx.overlap
        w13c, w2c = w13.contiguous(), w2.contiguous()
        ss, sc = p["seg_start"], p["seg_count"]
        with trace.phase("ep.bwd.dispatch"):
            if ov:
                dgs, events = _dispatch_side(fctx, p, dyc, mode, ep, backward=True)
            else:
                dgs = _dispatch(fctx, p, dyc, mode, ep, backward=True)
        xin, dout = fctx.section(XIN), fctx.section(DOUT)
        # d(act) = dout @ w2^T never reaches memory: the GEMM's epilogue applies the SwiGLU
        # backward to its tile and writes d[gate | up]
        dh13 = torch.empty_like(h13)
        with trace.phase("ep.bwd.experts"):
            lib.zero_pad_rows(dout, ss, sc, SEG_ALIGN)
            if ov:
                cur = torch.cuda.current_stream(fctx.device) if events else None
                dw2 = torch.empty_like(w2c)
                nch = len(fctx.chunks)
                for i, (lo, hi) in enumerate(fctx.chunks):
                    if cur is not None:
                        cur.wait_event(events[i])
                    lib.grouped_gemm_ex(dout, w2c[lo:hi], dh13, h13, ss[lo:hi], sc[lo:hi], 1, 3,
                                        fctx.arena, FK_B_DATA, first, n, flag_value(ep, i, nch),
                                        SEG_ALIGN)
                    if i == nch - 1:
                        fctx.mark_link_quiet()      # every dY row has arrived; two wgrad GEMMs follow
                    lib.grouped_wgrad_out(act, dout, dw2, lo, ss[lo:hi], sc[lo:hi], 0, SEG_ALIGN)
                dw13 = lib.grouped_wgrad(xin, dh13, ss, sc, 0, SEG_ALIGN)
                base, slots = ((fctx.dret_base, fctx.ret_slots) if mode == "one_hop"
                               else (fctx.dret2_base, fctx.ret2_slots))
                lib.grouped_gemm_scatter(dh13, w13c, ss, sc, 1, fctx.row_map, base, slots)
                LIVE["overlap_bwd"] += 1
            else:
                lib.grouped_gemm_ex(dout, w2c, dh13, h13, ss, sc, 1, 3, fctx.arena, FK_B_DATA,
                                    first, n, flag_value(ep, 0, 1), SEG_ALIGN)
                fctx.mark_link_quiet()
                dw2 = lib.grouped_wgrad(act, dout, ss, sc, 0, SEG_ALIGN)
                dw13 = lib.grouped_wgrad(xin, dh13, ss, sc, 0, SEG_ALIGN)
                lib.grouped_gemm_ex(dh13, w13c, fctx.section(DXS), None, ss, sc, 1, 0, None, 0, 0,
                                    0, ep, SEG_ALIGN)
        with trace.phase("ep.bwd.combine"):
            _signal_out(fctx, mode, FK_B_OUT, ep, dyc)
            dx = _combine(fctx, p, mode, ep, src=DXS, use_gate=False, backward=True)
            if mode == "two_hop":
                dgs = lib.origin_pull_dgate(fctx.arena, p["es"], p["rowa"], FK_B_DG, ep)
        dgates = torch.zeros_like(dgs).scatter_(1, p["cols"].long(), dgs).to(ctx.gate_dtype)
        LIVE[f"{mode}_bwd"] += 1
        fctx.release(ctx)
        return dx, dgates, dw13, dw2, None, None, None, None


def fused_moe_forward(fctx: FusedEPContext, x, idx, gates, w13, w2, *, mode: str,
                      capacity_factor=None, tokens_global=None):
    """Routed-expert output for this rank's tokens over the fused transport.

    ``capacity_factor`` bounds the rows every expert accepts to ``ceil(cf * tokens_global * k /
    E)`` (``tokens_global`` defaults to this rank's tokens times the world size); picks beyond
    the bound, in canonical order (source rank, then token), are dropped on the device: they are
    not sent, occupy no GEMM row and receive no gradient -- the semantics of
    ``layer.apply_capacity`` without its host-side counts exchange."""
    if mode == "two_hop" and not fctx.two_hop_ok:
        mode = "one_hop"          # fewer than two groups (or groups != routing groups)
    fctx.check_mode(mode)
    if x.shape[0] > fctx.tokens:
        raise ValueError(f"{x.shape[0]} tokens exceed the context capacity {fctx.tokens}")
    if x.dtype != torch.bfloat16 or w13.dtype != torch.bfloat16:
        raise TypeError("the fused transport moves bf16 rows")
    cap = expert_capacity(capacity_factor, tokens_global or x.shape[0] * fctx.world, fctx.k,
                          fctx.E)
    return _FusedMoE.apply(x, gates, w13, w2, idx, fctx, mode, cap)


def pipeline_depth() -> int:
    """``TERRACE_EP_PIPELINE=n`` (default 1 = off): run the fused layer on ``n`` token slices."""
    return flag_int("TERRACE_EP_PIPELINE", 1, 1, 8)


class PipelinedFusedEP:
    """Token-sliced software pipeline over the fused transport: ``n`` independent arenas, each
    slice of the tokens runs plan -> push -> GEMMs -> combine on its own CUDA stream, so that the
    dispatch and combine of one slice overlap the expert GEMMs of another.  The kernels are the
    unchanged ones of the unsliced path.  (The default schedule already overlaps chunk by chunk
    inside one arena; slicing by tokens is the alternative that needs no scattering epilogue.)

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

    def status_tensor(self) -> torch.Tensor:
        return self.ctxs[0].status_tensor()

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


def run_fused(ctx, x, idx, gates, w13, w2, *, mode: str, capacity_factor=None,
              tokens_global=None):
    if isinstance(ctx, PipelinedFusedEP):
        if capacity_factor is not None:
            raise ValueError("the token pipeline does not bound expert capacity: a slice sees "
                             "only its own tokens")
        return ctx.forward(x, idx, gates, w13, w2, mode=mode)
    return fused_moe_forward(ctx, x, idx, gates, w13, w2, mode=mode,
                             capacity_factor=capacity_factor, tokens_global=tokens_global)


@torch.no_grad()
def fused_dispatch_combine(fctx: FusedEPContext, x, idx, gates, *, mode: str):
    """Dispatch immediately followed by combine (rows echo back unchanged, gate-weighted): the
    communication-only measurement.  The rows come back by remote reads of the owners' input
    sections, whatever the context's schedule (no GEMM runs whose epilogue could return them)."""
    if isinstance(fctx, PipelinedFusedEP):      # slice after slice on the caller's stream
        return torch.cat([fused_dispatch_combine(c, x[lo:hi], idx[lo:hi], gates[lo:hi], mode=mode)
                          for (lo, hi), c in zip(fctx.bounds(x.shape[0]), fctx.ctxs)], dim=0)
    if mode == "two_hop" and not fctx.two_hop_ok:
        mode = "one_hop"
    fctx.check_mode(mode)
    fctx.check_free()
    ep = fctx.next_epoch()
    p = _plan(fctx, idx, gates, mode, ep)
    _dispatch(fctx, p, x.contiguous(), mode, ep)
    _signal_out(fctx, mode, FK_OUT, ep, x, wait_kind=FK_DATA)
    LIVE["echo"] += 1
    return _combine(fctx, p, mode, ep, src=XIN, use_gate=True, backward=False, pull=True)
