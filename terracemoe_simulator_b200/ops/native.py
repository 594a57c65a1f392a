"""Autograd wrappers around the sm_100a compute kernels.

Every wrapper has a ``*_supported`` predicate (dtype / alignment limits of the kernel); callers
fall back to the PyTorch expression when it says no.  All backward passes are hand-written and
call the same kernels (dgrad = grouped GEMM with the K-major weight view, wgrad = the
transposed-operand GEMM), so no library GEMM runs on these paths.

What the wrappers replace in the reference: ``rmsnorm`` (terrace/model.py:46-47), the router
chain (terrace/routing.py:132-134), ``nn.Linear`` / ``SwiGLU`` (terrace/layer.py:19-27), the
grouped matmul and its autograd (terrace/layer.py:30-74) and the permute / expert / un-permute
chain of ``TerracedMoE._experts_grouped`` (terrace/layer.py:101-112).
"""
from __future__ import annotations

import torch

LIVE = {"rmsnorm": 0, "route": 0, "route_fused": 0, "rope_split": 0, "linear": 0, "swiglu_ffn": 0, "grouped_mm": 0,
        "moe_experts_local": 0, "attention": 0}


# Kernel launches issued through this module since the last reset (bench.py reports it).
LAUNCHES = [0]


class _Counted:
    """Proxy of ``torch.ops.terrace`` that counts kernel launches per op call."""
    _PER_CALL = {"rmsnorm_fwd": 1, "rmsnorm_bwd": 1, "route_select": 1, "route_select_bwd": 1, "route_fused": 1, "rope_split": 1,
                 "rope_merge": 1,
                 "moe_plan": 3, "moe_scatter_rows": 1, "moe_combine": 1, "moe_combine_bwd": 1,
                 "swiglu_bwd": 1, "grouped_gemm": 1, "grouped_wgrad": 1, "passthrough": 1,
                 "zero_pad_rows": 1,
                 "k1_arrival": 3, "k2_pack": 3, "ep_plan_pass1": 1, "ep_plan": 1, "ep_push": 1,
                 "ep_signal": 1, "ep_pull_combine": 1, "hopa_rank": 1, "hopa_push": 1,
                 "arrival_push": 1, "arrival_combine": 1, "origin_combine": 1,
                 "origin_pull_dgate": 1, "grouped_gemm_ex": 1, "attn_fwd": 1, "attn_bwd": 3,
                 "grouped_wgrad_out": 1, "grouped_gemm_scatter": 1}

    def __getattr__(self, name):
        fn = getattr(torch.ops.terrace, name)
        n = self._PER_CALL.get(name, 0)
        if n == 0:
            return fn

        def call(*a, **kw):
            LAUNCHES[0] += n
            return fn(*a, **kw)
        return call


_COUNTED = _Counted()


def _lib():
    return _COUNTED


def _bf16_cuda(*ts) -> bool:
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts)


def take_status(device=None) -> int:
    """Read-and-clear the device status word (host sync). Non-zero = a kernel contained a
    problem: 1/2/3 pipeline wait timeouts, 4 flag timeout, 5 bad row index, 6 counts timeout."""
    if device is None:
        device = torch.cuda.current_device()
    code = int(_lib().take_status(int(device)))
    return code or int(torch.ops.terrace.symm_take_status(int(device)))


# ---------------------------------------------------------------------------------------------
# RMSNorm
# ---------------------------------------------------------------------------------------------
def rmsnorm_supported(x, w) -> bool:
    return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and w.dtype == x.dtype
            and x.shape[-1] == w.numel())


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        xc = x.contiguous()
        y, rstd = _lib().rmsnorm_fwd(xc, w.contiguous(), float(eps))
        ctx.save_for_backward(xc, w, rstd)
        LIVE["rmsnorm"] += 1
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dx, part = _lib().rmsnorm_bwd(x, w.contiguous(), dy.contiguous(), rstd)
        return dx, part.sum(dim=0).to(w.dtype), None


def rmsnorm(x, w, eps=1e-5):
    return _RMSNorm.apply(x, w, eps)


# ---------------------------------------------------------------------------------------------
# dense GEMMs (single group)
# ---------------------------------------------------------------------------------------------
def _one_segment(rows: int, device):
    start = torch.zeros(1, dtype=torch.int32, device=device)
    count = torch.full((1,), rows, dtype=torch.int32, device=device)
    return start, count


def _aligned(*dims) -> bool:
    return all(d % 8 == 0 for d in dims)


def dense_supported(x, w) -> bool:
    return (_bf16_cuda(x, w) and x.shape[-1] == w.shape[-1] and
            _aligned(x.shape[-1], w.shape[0]) and min(x.shape[-1], w.shape[0]) >= 64)


class _Linear(torch.autograd.Function):
    """y = x @ w^T with w [out, in] (the ``nn.Linear`` layout)."""

    @staticmethod
    def forward(ctx, x, w):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        s, c = _one_segment(x2.shape[0], x.device)
        y, _ = _lib().grouped_gemm(x2, w.contiguous().unsqueeze(0), s, c, 1, 0, False, 0)
        ctx.save_for_backward(x2, w, s, c)
        ctx.lead = x.shape[:-1]
        LIVE["linear"] += 1
        return y.view(*ctx.lead, w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, s, c = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx, _ = _lib().grouped_gemm(dy2, w.contiguous().unsqueeze(0), s, c, 0, 0, False, 0)
            dx = dx.view(*ctx.lead, w.shape[1])
        if ctx.needs_input_grad[1]:
            dw = _lib().grouped_wgrad(dy2, x2, s, c, 0)[0]
        return dx, dw


def linear(x, w):
    return _Linear.apply(x, w)


class _SwiGLUFFN(torch.autograd.Function):
    """``w2(silu(a) * b)`` with ``[a | b] = w13(x)``; weights in ``nn.Linear`` layout
    (``w13 [2i, h]``, ``w2 [h, i]``).  SiLU*mul is fused into the first GEMM's epilogue."""

    @staticmethod
    def forward(ctx, x, w13, w2):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        s, c = _one_segment(x2.shape[0], x.device)
        need = any(ctx.needs_input_grad)
        act, h13 = _lib().grouped_gemm(x2, w13.contiguous().unsqueeze(0), s, c, 1, 1, need, 0)
        y, _ = _lib().grouped_gemm(act, w2.contiguous().unsqueeze(0), s, c, 1, 0, False, 0)
        ctx.save_for_backward(x2, w13, w2, h13, act, s, c)
        ctx.lead = x.shape[:-1]
        LIVE["swiglu_ffn"] += 1
        return y.view(*ctx.lead, w2.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w13, w2, h13, act, s, c = ctx.saved_tensors
        lib = _lib()
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        # d(act) GEMM with the SwiGLU backward in its epilogue: writes d[gate | up] directly
        dh13 = torch.empty_like(h13)
        lib.grouped_gemm_ex(dy2, w2.contiguous().unsqueeze(0), dh13, h13, s, c, 0, 3, None, 0, 0,
                            0, 0, 0)
        dw2 = lib.grouped_wgrad(dy2, act, s, c, 0)[0]
        dx, _ = lib.grouped_gemm(dh13, w13.contiguous().unsqueeze(0), s, c, 0, 0, False, 0)
        dw13 = lib.grouped_wgrad(dh13, x2, s, c, 0)[0]
        return dx.view(*ctx.lead, x2.shape[1]), dw13, dw2


def swiglu_ffn(x, w13, w2):
    return _SwiGLUFFN.apply(x, w13, w2)


# ---------------------------------------------------------------------------------------------
# grouped matmul (rows pre-sorted by group)
# ---------------------------------------------------------------------------------------------
def grouped_supported(x, w) -> bool:
    return (_bf16_cuda(x, w) and w.dim() == 3 and x.dim() == 2 and x.shape[1] == w.shape[1]
            and _aligned(w.shape[1], w.shape[2]) and min(w.shape[1], w.shape[2]) >= 64
            and w.shape[0] <= 1024)


def segments_from_counts(counts: torch.Tensor):
    c = counts.to(torch.int32)
    start = (torch.cumsum(c, 0, dtype=torch.int32) - c).contiguous()
    return start, c.contiguous()


class _GroupedMM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, counts):
        s, c = segments_from_counts(counts)
        xc = x.contiguous()
        y, _ = _lib().grouped_gemm(xc, w.contiguous(), s, c, 0, 0, False, 0)
        ctx.save_for_backward(xc, w, s, c)
        LIVE["grouped_mm"] += 1
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, s, c = ctx.saved_tensors
        dyc = dy.contiguous()
        dx, _ = _lib().grouped_gemm(dyc, w.contiguous(), s, c, 1, 0, False, 0)
        dw = _lib().grouped_wgrad(x, dyc, s, c, 0)
        return dx, dw, None


def grouped_mm_native(x, w, counts):
    return _GroupedMM.apply(x, w, counts)


# ---------------------------------------------------------------------------------------------
# router
# ---------------------------------------------------------------------------------------------
def router_supported(cfg, hidden) -> bool:
    g = cfg.group_size
    return (hidden.is_cuda and cfg.n_experts <= 512 and cfg.n_groups <= 64 and g <= 512
            and cfg.top_k <= 32)


class _RouteSelect(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, n_groups, top_k, top_groups, pool):
        idx, gates, gidx, load, aff = _lib().route_select(
            logits.float().contiguous(), bias.float().contiguous(), n_groups, top_k, top_groups,
            pool)
        ctx.save_for_backward(gates, aff, idx)
        ctx.E = logits.shape[1]
        ctx.in_dtype = logits.dtype
        ctx.mark_non_differentiable(idx, gidx, load)
        LIVE["route"] += 1
        return idx, gates, gidx, load

    @staticmethod
    def backward(ctx, _di, dgates, _dg, _dl):
        gates, aff, idx = ctx.saved_tensors
        dlogits = _lib().route_select_bwd(dgates.contiguous(), gates, aff, idx, ctx.E)
        return dlogits.to(ctx.in_dtype), None, None, None, None, None


def route_from_logits(logits, bias, cfg):
    """T-Route (mode ``full``) from router logits: ``(idx, gates fp32, group_idx, load)``."""
    return _RouteSelect.apply(logits, bias, cfg.n_groups, cfg.top_k, cfg.top_groups,
                              cfg.group_score_pool)


class _RouteFused(torch.autograd.Function):
    """Router GEMM and T-Route selection (mode ``full``, sigmoid scores) in one launch; the
    logits stay in TMEM.  Backward: the gate gradients go back through the renormalisation and
    the sigmoid to ``dlogits`` (one launch), then through the router GEMM to the hidden states
    and the router weight (two launches of the dense kernels)."""

    @staticmethod
    def forward(ctx, hidden, weight, bias, n_groups, top_k, top_groups, pool):
        h2, w = hidden.contiguous(), weight.contiguous()
        idx, gates, gidx, load, aff = _lib().route_fused(
            h2, w, bias.float().contiguous(), n_groups, top_k, top_groups, pool)
        ctx.save_for_backward(h2, w, gates, aff, idx)
        ctx.mark_non_differentiable(idx, gidx, load)
        LIVE["route_fused"] += 1
        return idx, gates, gidx, load

    @staticmethod
    def backward(ctx, _di, dgates, _dg, _dl):
        h2, w, gates, aff, idx = ctx.saved_tensors
        lib = _lib()
        dlogits = lib.route_select_bwd(dgates.contiguous(), gates, aff, idx, w.shape[0])
        dl = dlogits.to(h2.dtype)
        s, c = _one_segment(h2.shape[0], h2.device)
        dh = dw = None
        if ctx.needs_input_grad[0]:
            dh, _ = lib.grouped_gemm(dl, w.unsqueeze(0), s, c, 0, 0, False, 0)
        if ctx.needs_input_grad[1]:
            dw = lib.grouped_wgrad(dl, h2, s, c, 0)[0]
        return dh, dw, None, None, None, None, None


def route_fused_supported(cfg, hidden, weight) -> bool:
    """One-launch router: bf16 hidden states and weight, at most 128 experts (multiple of 16)."""
    if not (_bf16_cuda(hidden, weight) and hidden.shape[-1] == weight.shape[-1]):
        return False
    return bool(torch.ops.terrace.route_fused_supported(
        cfg.n_experts, hidden.shape[-1], cfg.n_groups, cfg.top_k, cfg.top_groups))


def route_hidden(hidden, weight, bias, cfg):
    """T-Route (mode ``full``) from hidden states ``[T, H]``: ``(idx, gates fp32, group_idx,
    load)``.  One fused launch when the geometry allows, else router GEMM + select kernel."""
    h2 = hidden.reshape(-1, hidden.shape[-1])
    if route_fused_supported(cfg, h2, weight):
        return _RouteFused.apply(h2, weight, bias, cfg.n_groups, cfg.top_k, cfg.top_groups,
                                 cfg.group_score_pool)
    if dense_supported(h2, weight):
        logits = linear(h2, weight)
    else:
        logits = h2 @ weight.t().to(h2.dtype)
    return route_from_logits(logits, bias, cfg)


def fused_route(hidden, weight, bias, cfg):
    idx, gates, gidx, _load = route_hidden(hidden, weight, bias, cfg)
    return idx, gates, gidx


# ---------------------------------------------------------------------------------------------
# local routed experts: plan -> scatter -> grouped SwiGLU GEMMs -> deterministic combine
# ---------------------------------------------------------------------------------------------
def moe_local_supported(x, w13, w2) -> bool:
    return (_bf16_cuda(x, w13, w2) and _aligned(w13.shape[1], w13.shape[2] // 2, w2.shape[2])
            and min(w13.shape[1], w13.shape[2] // 2) >= 64 and w13.shape[0] <= 1024)


SEG_ALIGN = 64      # expert segments start on multiples of 64 rows; padding rows hold zeros


class _MoELocal(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, expert_idx, gates, w13, w2, group_size):
        lib = _lib()
        E = w13.shape[0]
        T, k = expert_idx.shape
        xc = x.contiguous()
        rows_cap = T * k + E * (SEG_ALIGN - 1)
        es, gs, cols, pos, seg_start, seg_count = lib.moe_plan(
            expert_idx.contiguous(), gates.detach().float().contiguous(), E, SEG_ALIGN)
        xs = lib.moe_scatter_rows(xc, pos, rows_cap)
        need = any(ctx.needs_input_grad)
        if need:
            lib.zero_pad_rows(xs, seg_start, seg_count, SEG_ALIGN)   # wgrad reads the padding
        act, h13 = lib.grouped_gemm(xs, w13.contiguous(), seg_start, seg_count, 0, 1, need, 0,
                                    SEG_ALIGN)
        out, _ = lib.grouped_gemm(act, w2.contiguous(), seg_start, seg_count, 0, 0, False, 0,
                                  SEG_ALIGN)
        y = lib.moe_combine(out, pos, es, gs, group_size)
        ctx.save_for_backward(xs, h13, act, out, pos, es, gs, cols, seg_start, seg_count, w13, w2)
        ctx.group_size = group_size
        ctx.gate_dtype = gates.dtype
        LIVE["moe_experts_local"] += 1
        return y

    @staticmethod
    def backward(ctx, dy):
        xs, h13, act, out, pos, es, gs, cols, seg_start, seg_count, w13, w2 = ctx.saved_tensors
        lib = _lib()
        A = SEG_ALIGN
        dout, dgs = lib.moe_combine_bwd(dy.contiguous(), out, pos, gs, True)
        lib.zero_pad_rows(dout, seg_start, seg_count, A)
        dh13 = torch.empty_like(h13)        # d(act) GEMM + SwiGLU backward in one kernel
        lib.grouped_gemm_ex(dout, w2.contiguous(), dh13, h13, seg_start, seg_count, 1, 3, None, 0,
                            0, 0, 0, A)
        dw2 = lib.grouped_wgrad(act, dout, seg_start, seg_count, 0, A)
        dxs, _ = lib.grouped_gemm(dh13, w13.contiguous(), seg_start, seg_count, 1, 0, False, 0, A)
        dw13 = lib.grouped_wgrad(xs, dh13, seg_start, seg_count, 0, A)
        dx = lib.moe_combine(dxs, pos, es, None, ctx.group_size)
        dgates = torch.zeros_like(dgs).scatter_(1, cols.long(), dgs).to(ctx.gate_dtype)
        return dx, None, dgates, dw13, dw2, None


def moe_experts_local(x, expert_idx, gates, w13, w2, group_size: int | None = None):
    """Routed-expert output ``y[T, H]`` for local experts ``w13[E, H, 2d]``, ``w2[E, d, H]``."""
    if group_size is None:
        group_size = w13.shape[0]
    return _MoELocal.apply(x, expert_idx, gates, w13, w2, int(group_size))


# ---------------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------------
class _Attention(torch.autograd.Function):
    """softmax(scale * q k^T (+ causal mask)) v on q, k, v [B, H, S, D] through the tcgen05
    attention kernels (forward saves the log-sum-exp; backward recomputes the probabilities)."""

    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o, lse = _lib().attn_fwd(q, k, v, bool(causal), float(scale))
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.causal, ctx.scale = bool(causal), float(scale)
        LIVE["attention"] += 1
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = _lib().attn_bwd(q, k, v, o, d_o.contiguous(), lse, ctx.causal, ctx.scale)
        return dq, dk, dv, None, None


class _RopeSplit(torch.autograd.Function):
    """``qkv [B, T, 3 * nh * hd] -> q, k, v [B, nh, T, hd]`` with interleaved RoPE applied to q and
    k, in one pass (the backward is the same kernel run the other way)."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, n_heads):
        q, k, v = _lib().rope_split(qkv.contiguous(), cos, sin, int(n_heads))
        ctx.save_for_backward(cos, sin)
        LIVE["rope_split"] += 1
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        cos, sin = ctx.saved_tensors
        return (_lib().rope_merge(dq.contiguous(), dk.contiguous(), dv.contiguous(), cos, sin),
                None, None, None)


def rope_split_supported(qkv, n_heads: int) -> bool:
    return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.dim() == 3
            and qkv.shape[-1] % (3 * n_heads) == 0 and (qkv.shape[-1] // (3 * n_heads)) % 8 == 0)


def rope_split(qkv, cos, sin, n_heads: int):
    """``cos`` / ``sin``: the model's RoPE tables ``[..., T, hd / 2]`` (any leading ones)."""
    T, half = qkv.shape[1], qkv.shape[-1] // (3 * n_heads) // 2
    c = cos.reshape(-1, half)[:T].float().contiguous()
    s = sin.reshape(-1, half)[:T].float().contiguous()
    return _RopeSplit.apply(qkv, c, s, n_heads)


def attention_shape_supported(q, causal: bool = True) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.dim() == 4
            and (causal or q.shape[-2] % 128 == 0) and q.shape[-1] in (64, 128))


def attention(q, k, v, causal: bool = True, scale: float | None = None):
    """Self-attention on [B, H, S, D] bf16 tensors, D 64 or 128.  The kernels work on blocks of
    128 positions; a causal sequence of any other length is padded with zero rows at the end,
    which the mask hides from every real query (the padded queries' outputs are dropped and
    receive zero gradient), so the result is exact.  Without a mask S must be a multiple of 128."""
    if scale is None:
        scale = q.shape[-1] ** -0.5
    S = q.shape[-2]
    pad = (-S) % 128
    if pad == 0:
        return _Attention.apply(q, k, v, causal, scale)
    if not causal:
        raise ValueError("attention without a causal mask needs a sequence length that is a "
                         "multiple of 128")
    qp, kp, vp = (torch.nn.functional.pad(t, (0, 0, 0, pad)) for t in (q, k, v))
    return _Attention.apply(qp, kp, vp, True, scale)[..., :S, :]


def attention_supported(x, n_heads) -> bool:
    """Can the attention of a [B, T, dim] bf16 activation with n_heads heads run natively?
    ``TERRACE_ATTENTION=sdpa`` keeps the model on torch's scaled_dot_product_attention (the
    library kernel is about twice as fast as the kernels of this package at head width 128)."""
    from ..utils.flags import flag_choice
    if flag_choice("TERRACE_ATTENTION", ("native", "sdpa"), "native") == "sdpa":
        return False
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 3):
        return False
    hd = x.shape[-1] // n_heads
    return hd in (64, 128)           # any length: the causal wrapper pads to blocks of 128
