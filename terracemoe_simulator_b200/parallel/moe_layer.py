"""Expert-parallel MoE layer: T-Route router + routed experts over one of four transports.

``mode``      ``fused``   transport
``local``     --          all experts on this GPU (permute, grouped GEMMs, combine kernels)
``one_hop``   False       ``torch.distributed`` all-to-all (``parallel/ep.py``; the baseline arm)
``one_hop``   True        fused peer-memory dispatch / combine kernels (``parallel/fused.py``)
``two_hop``   False       T-A2A over ``torch.distributed`` (``parallel/ta2a.py``)
``two_hop``   True        fused T-A2A: Hop A push to the group representative, Hop B push into the
                          owner's expert-sorted GEMM input, gate-weighted pull combine

The reference has no EP-aware module: its ``TerracedMoE`` is single device and the EP paths are
bare functions (``terrace/ep_dist.py:82``, ``terrace/ta2a_fwd.py:445``).  ``EPTerracedMoE`` keeps
``TerracedMoE``'s parameters, stats dict and in-forward bias update (``terrace/layer.py:119-130``)
and holds only this rank's expert shard ``w13[epr, h, 2d]`` / ``w2[epr, d, h]``; the router and
the shared expert are replicated.  The router's expert load is summed over ranks before the
bias update so every replica takes the same step.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..layer import SwiGLU, apply_capacity
from ..routing import Router, TRouteConfig, expert_load, t_route, update_bias_
from .ep import ep_moe_forward
from .ta2a import init_ta2a_groups, ta2a_moe_forward

EP_MODES = ("local", "one_hop", "two_hop")


def _route(x, router_w, bias, cfg):
    """Router logits + T-Route; native kernels when available."""
    if x.is_cuda and ops.custom_ops_enabled() and ops.router_supported(cfg, x):
        return ops.route_hidden(x, router_w, bias, cfg)
    aff = torch.sigmoid((x @ router_w.t().to(x.dtype)).float())
    idx, gates, gidx = t_route(aff, bias.float(), cfg, "full")
    return idx, gates, gidx, expert_load(idx, cfg.n_experts)


def routed_experts(x, idx, gates, w13, w2, cfg: TRouteConfig, *, mode: str, world: int, rpn: int,
                   fused: bool, ctx=None, capacity_factor=None):
    """Dispatch -> expert SwiGLU -> combine for this rank's tokens, on the chosen transport.
    ``capacity_factor`` is applied on the device by the fused transport only; the other
    transports expect gates that ``layer.apply_capacity`` has already zeroed."""
    if mode not in EP_MODES:
        raise ValueError(f"unknown EP mode {mode!r}; expected one of {EP_MODES}")
    E = cfg.n_experts
    if mode == "local" or world == 1:
        if x.is_cuda and ops.custom_ops_enabled() and ops.moe_local_supported(x, w13, w2):
            return ops.moe_experts_local(x, idx, gates, w13, w2, cfg.group_size)
        # PyTorch path: canonical tree through the one-hop code with a single rank is not
        # available without a process group, so use the plain grouped formulation
        from ..layer import grouped_mm
        T, k = idx.shape
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        tok = torch.div(order, k, rounding_mode="floor")
        counts = torch.zeros(E, dtype=torch.int64, device=x.device).scatter_add_(
            0, flat, torch.ones_like(flat))
        a, b = grouped_mm(x[tok], w13, counts).chunk(2, dim=-1)
        out = grouped_mm(torch.nn.functional.silu(a) * b, w2, counts)
        w = gates.reshape(-1)[order].unsqueeze(-1).to(out.dtype)
        return torch.zeros_like(x).index_add(0, tok, w * out)
    if fused:
        from . import fused as fz
        return fz.run_fused(ctx, x, idx, gates, w13, w2, mode=mode,
                            capacity_factor=capacity_factor)
    if mode == "one_hop":
        return ep_moe_forward(x, idx, gates, w13, w2, world, E, rpn=rpn)
    return ta2a_moe_forward(x, idx, gates, w13, w2, world, E, rpn=rpn, groups_m=cfg.top_groups)


class MoELayerRunner:
    """Functional MoE layer ``(x, router_w, w13_shard, w2_shard) -> y`` used by the benchmarks
    and the tests; owns the per-layer communication context (process groups or the symmetric
    arena of the fused transport)."""

    def __init__(self, cfg: TRouteConfig, hidden: int, d_expert: int, tokens: int, *, world: int,
                 rank: int, rpn: int, mode: str, fused: bool, device, overlap=None):
        """``overlap``: schedule of the fused transport (None = ``TERRACE_EP_OVERLAP``, default
        on; False = the remote-read schedule, the A/B arm)."""
        if mode not in EP_MODES:
            raise ValueError(f"unknown EP mode {mode!r}; expected one of {EP_MODES}")
        self.cfg, self.world, self.rank, self.rpn = cfg, world, rank, rpn
        self.mode, self.fused = mode, fused and world > 1
        self.hidden, self.d_expert, self.tokens = hidden, d_expert, tokens
        self.device = device
        self.bias = torch.zeros(cfg.n_experts, device=device)
        self.ctx = None
        if world > 1 and mode == "two_hop" and not self.fused:
            init_ta2a_groups(world, rpn)
        if self.fused:
            from . import fused as fz
            self.ctx = fz.make_context(cfg, hidden, d_expert, tokens, world=world, rank=rank,
                                       rpn=rpn, device=device, overlap=overlap)

    def __call__(self, x, router_w, w13, w2):
        idx, gates, _gidx, _load = _route(x, router_w, self.bias, self.cfg)
        return routed_experts(x, idx, gates, w13, w2, self.cfg, mode=self.mode, world=self.world,
                              rpn=self.rpn, fused=self.fused, ctx=self.ctx)

    @torch.no_grad()
    def time_dispatch_combine(self, x, steps: int, warmup: int) -> float:
        """Dispatch + combine only (no expert compute): rows go out and come straight back.
        Device-timed, max over ranks, microseconds per call."""
        cfg = self.cfg
        g = torch.Generator(device="cpu").manual_seed(7 + self.rank)
        aff = torch.rand(x.shape[0], cfg.n_experts, generator=g).to(x.device)
        idx, gates, _ = t_route(aff, self.bias, cfg, "full")
        fn = self._dispatch_combine_fn(x, idx, gates)
        if fn is None:
            return float("nan")
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            fn()
        t1.record()
        torch.cuda.synchronize()
        us = torch.tensor([t0.elapsed_time(t1) * 1e3 / steps], device=x.device)
        if self.world > 1:
            dist.all_reduce(us, op=dist.ReduceOp.MAX)
        return us.item()

    def _dispatch_combine_fn(self, x, idx, gates):
        lib = torch.ops.terrace
        E, cfg = self.cfg.n_experts, self.cfg
        T, k = idx.shape
        if self.mode == "local" or self.world == 1:
            if not (ops.custom_ops_enabled() and x.dtype == torch.bfloat16):
                return None
            g32 = gates.float().contiguous()

            def fn():
                es, gs, cols, pos, s0, c0 = lib.moe_plan(idx, g32, E, 1)
                xs = lib.moe_scatter_rows(x, pos, T * k)
                return lib.moe_combine(xs, pos, es, gs, cfg.group_size)
            return fn
        if self.fused:
            from . import fused as fz
            return lambda: fz.fused_dispatch_combine(self.ctx, x, idx, gates, mode=self.mode)
        # torch.distributed arm: the same exchange with the expert compute replaced by identity

        def echo(rows, *_):
            return rows

        def fn():
            if self.mode == "one_hop":
                return ep_moe_forward(x, idx, gates, None, None, self.world, E, rpn=self.rpn,
                                      experts_fn=echo)
            return ta2a_moe_forward(x, idx, gates, None, None, self.world, E, rpn=self.rpn,
                                    groups_m=cfg.top_groups, experts_fn=echo)
        return fn


class EPTerracedMoE(nn.Module):
    """``TerracedMoE`` whose routed experts are sharded over the default process group."""

    def __init__(self, hidden: int, d_expert: int, d_shared: int, cfg: TRouteConfig,
                 n_shared: int = 1, bias_gamma: float = 1e-3, *, mode: str = "one_hop",
                 rpn: int = 1, fused: bool = False, capacity_factor: float | None = None,
                 tokens_hint: int | None = None, row_capacity_factor: float = 2.0):
        super().__init__()
        if mode not in EP_MODES:
            raise ValueError(f"unknown EP mode {mode!r}; expected one of {EP_MODES}")
        self.cfg, self.bias_gamma, self.mode, self.rpn, self.fused = cfg, bias_gamma, mode, rpn, fused
        self.capacity_factor = capacity_factor
        self.routing_mode = "full"
        self.expert_backend = "native"
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        if cfg.n_experts % self.world:
            raise ValueError(f"n_experts={cfg.n_experts} not divisible by world={self.world}")
        epr = cfg.n_experts // self.world
        self.hidden, self.d_expert, self.tokens_hint = hidden, d_expert, tokens_hint
        # rows an expert owner's arena holds, as a multiple of tokens * top_k: 1.0 is perfectly
        # balanced routing, `world` the worst case.  A step that exceeds it skips the overflowing
        # rows and raises the device status word (stats["ep_status"], `check_status`).
        self.row_capacity_factor = row_capacity_factor
        self.router = Router(hidden, cfg)
        self.shared = SwiGLU(hidden, n_shared * d_shared)
        self.w13 = nn.Parameter(torch.empty(epr, hidden, 2 * d_expert))
        self.w2 = nn.Parameter(torch.empty(epr, d_expert, hidden))
        nn.init.normal_(self.w13, std=hidden ** -0.5)
        nn.init.normal_(self.w2, std=d_expert ** -0.5)
        self._ctx = None
        if self.world > 1 and mode == "two_hop" and not fused:
            init_ta2a_groups(self.world, rpn)

    def _context(self, tokens: int, device):
        """The fused transport's arena, created at the first call for the largest token count
        of any rank (one host synchronisation, once).  Growing it later is a collective decision:
        every rank calls :meth:`reserve` between steps."""
        if not self.fused or self.world == 1:
            return None
        if self._ctx is None:
            want = torch.tensor([max(tokens, self.tokens_hint or 0)], device=device)
            dist.all_reduce(want, op=dist.ReduceOp.MAX)
            self._build_context(int(want.item()), device)
        elif self._ctx.tokens < tokens:
            raise RuntimeError(
                f"{tokens} tokens exceed the arena sized for {self._ctx.tokens}: call "
                "reserve(tokens) on every rank between steps (or pass tokens_hint)")
        return self._ctx

    def _build_context(self, tokens: int, device):
        from . import fused as fz
        self._ctx = fz.make_context(self.cfg, self.hidden, self.d_expert, tokens,
                                    world=self.world, rank=self.rank, rpn=self.rpn, device=device,
                                    row_capacity_factor=self.row_capacity_factor,
                                    modes=(self.mode,) if self.mode in ("one_hop", "two_hop") else None)

    def reserve(self, tokens: int, device=None) -> None:
        """Collective: size the arena for ``tokens`` tokens per rank.  The old arena's peer
        mappings are closed and, after a barrier (no rank frees memory a peer still maps), a new
        one is allocated and exchanged."""
        if not self.fused or self.world == 1:
            return
        device = device or self.w13.device
        if self._ctx is not None:
            if self._ctx.tokens >= tokens:
                return
            torch.cuda.synchronize(device)
            self._ctx.close()
            dist.barrier()
            self._ctx = None
        self._build_context(tokens, device)

    def link_quiet_event(self):
        """CUDA event at which the latest backward's NVLink traffic paused (see
        ``FusedEPContext.link_quiet_event``); None without a fused context or before the first
        backward.  A host-to-device copy for a later step should wait for it."""
        ctx = getattr(self, "_ctx", None)
        return getattr(ctx, "link_quiet_event", lambda: None)() if ctx is not None else None

    def check_status(self) -> int:
        """Read and clear the device status word (one host synchronisation); raises when a kernel
        reported a problem, e.g. routed rows beyond ``row_capacity_factor``."""
        code = ops.take_status(self.w13.device.index) if self.w13.is_cuda else 0
        if code:
            raise RuntimeError(f"expert-parallel kernels reported status {code} "
                               "(5 = a row fell outside its buffer: raise row_capacity_factor)")
        return code

    def forward(self, x: torch.Tensor):
        lead = x.shape[:-1]
        x = x.reshape(-1, x.shape[-1])
        if self.routing_mode != "full":
            raise ValueError("the expert-parallel layer routes with mode 'full' only")
        idx, gates, gidx, load = _route(x, self.router.weight, self.router.bias, self.cfg)
        gates_used = gates
        on_device = self.fused and self.world > 1      # the fused plan kernel applies the cap
        if self.capacity_factor is not None and not on_device:
            all_load = load.clone()
            prior = torch.zeros_like(load)
            if self.world > 1:
                gathered = [torch.zeros_like(load) for _ in range(self.world)]
                dist.all_gather(gathered, load)
                prior = sum(gathered[: self.rank], torch.zeros_like(load))
                all_load = sum(gathered)
            gates_used, _keep, _cap = apply_capacity(
                idx, gates, self.cfg.n_experts, self.capacity_factor,
                n_tokens_global=x.shape[0] * self.world, prior_counts=prior.long())
        y = routed_experts(x, idx, gates_used, self.w13, self.w2, self.cfg, mode=self.mode,
                           world=self.world, rpn=self.rpn, fused=self.fused,
                           ctx=self._context(x.shape[0], x.device),
                           capacity_factor=self.capacity_factor if on_device else None)
        if self.shared.w2.in_features > 0:
            y = y + self.shared(x)
        if self.training:
            total = load.detach().clone()
            if self.world > 1:
                dist.all_reduce(total)
            update_bias_(self.router.bias, total, self.bias_gamma)
        stats = {"expert_load": load, "group_idx": gidx, "gates": gates, "expert_idx": idx}
        if self._ctx is not None:       # device word, no synchronisation: read it a few steps late
            stats["ep_status"] = self._ctx.status_tensor()
        return y.reshape(*lead, -1), stats
