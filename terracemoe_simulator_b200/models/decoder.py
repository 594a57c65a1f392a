"""TerraceLM: pre-norm decoder with causal attention (interleaved-pair RoPE) and Terraced-MoE
feed-forward blocks, plus the differentiable balance aux loss.

Parity with the reference ``terrace/model.py``:
  * ``ModelArgs`` defaults           -> model.py:20-43
  * ``rmsnorm``                      -> model.py:46-47
  * ``Attention`` / ``_rope``        -> model.py:50-71
  * ``Block``                        -> model.py:74-102  (dense FFN = SwiGLU(dim, 4 dim))
  * ``TerraceLM`` forward contract   -> model.py:105-145 (logits,{}) | (loss, info dict)
  * ``_balance_aux``                 -> model.py:148-166 (E * sum f_i P_i, mean over MoE layers)

The state-dict key set equals the reference's, so checkpoints interchange.  Extra fields
(``moe_every_layer``, ``capacity_factor``, ``score_func``, ``ep_*``) default to the reference
behaviour.  With native ops enabled on a B200 the norms, attention, dense projections and
routed experts run through the sm_100a kernels; otherwise plain PyTorch ops.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..layer import HierarchicalMoE, SwiGLU, TerracedMoE
from ..routing import TRouteConfig


@dataclass
class ModelArgs:
    vocab: int = 32000
    dim: int = 512
    n_layers: int = 12
    n_heads: int = 8
    seq_len: int = 1024
    n_experts: int = 64
    n_groups: int = 16
    top_k: int = 4
    top_groups: int = 2
    d_expert: int = 512
    d_shared: int = 1024
    n_shared: int = 1
    dense_first: int = 1
    bias_gamma: float = 1e-3
    routing_mode: str = "full"
    balance_aux: float = 1e-3
    expert_backend: str = "loop"
    arch: str = "flat"
    d0: int = 256
    d1: int = 1024
    p_hard: float = 0.25
    # --- additions (defaults reproduce the reference) ---
    moe_every_layer: bool = False        # True: every block is MoE (no dense first/last layer)
    capacity_factor: float | None = None
    ep_mode: str = "local"               # local | one_hop | two_hop (expert-parallel layer)
    ep_rpn: int = 1                      # ranks per logical group for two_hop
    ep_fused: bool = False               # fused peer-memory kernels instead of NCCL all_to_all
    ce_chunk: int = 0                    # > 0: LM head + cross-entropy in chunks of that many tokens


class _ChunkedLMLoss(torch.autograd.Function):
    """Mean cross-entropy of ``h @ w.T`` against ``targets`` without ever holding the
    ``[tokens, vocab]`` logits: the head GEMM, the loss and their gradients are computed one token
    chunk at a time in the forward pass (weight gradient accumulated in fp32), the backward pass
    only scales.  Every chunk rounds its logits to the dtype of ``h`` exactly as the unchunked
    ``head`` + ``F.cross_entropy(logits.float())`` does, so the loss differs from it only by the
    order of the final sum.  At vocabulary 32000 and 32768 tokens the logits, their fp32 copy and
    the gradient are 10 GB that this path never allocates.  The reference computes the loss in
    one piece (``terrace/model.py:135-138``)."""

    @staticmethod
    def forward(ctx, h, w, targets, chunk):
        n = h.shape[0]
        dh = torch.empty_like(h)
        dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        total = torch.zeros((), dtype=torch.float32, device=h.device)
        for s in range(0, n, chunk):
            hc = h[s:s + chunk].detach().requires_grad_(True)
            wc = w.detach().requires_grad_(True)
            with torch.enable_grad():
                part = F.cross_entropy(F.linear(hc, wc).float(), targets[s:s + chunk],
                                       reduction="sum")
            gh, gw = torch.autograd.grad(part, (hc, wc))
            dh[s:s + chunk] = gh
            dw += gw
            total += part.detach()
        ctx.save_for_backward(dh, dw)
        ctx.n, ctx.w_dtype = n, w.dtype
        return total / n

    @staticmethod
    def backward(ctx, g):
        dh, dw = ctx.saved_tensors
        scale = g / ctx.n
        return dh * scale.to(dh.dtype), (dw * scale).to(ctx.w_dtype), None, None


def chunked_lm_loss(h: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, chunk: int):
    """``F.cross_entropy(F.linear(h, w).float(), targets)`` computed in token chunks."""
    if chunk <= 0:
        raise ValueError("chunk must be positive")
    return _ChunkedLMLoss.apply(h.reshape(-1, h.shape[-1]), w, targets.reshape(-1), int(chunk))


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    from .. import ops
    if x.is_cuda and ops.custom_ops_enabled() and ops.rmsnorm_supported(x, w):
        return ops.rmsnorm(x, w, eps)
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate interleaved (even, odd) pairs of the head dimension. x: [B, nh, T, hd]."""
    even, odd = x[..., 0::2], x[..., 1::2]
    return torch.stack((even * cos - odd * sin, even * sin + odd * cos), dim=-1).flatten(-2)


class Attention(nn.Module):
    def __init__(self, a: ModelArgs):
        super().__init__()
        self.nh, self.hd = a.n_heads, a.dim // a.n_heads
        self.wqkv = nn.Linear(a.dim, 3 * a.dim, bias=False)
        self.wo = nn.Linear(a.dim, a.dim, bias=False)
        self.register_buffer("qn", torch.ones(self.hd), persistent=False)

    def forward(self, x, cos, sin):
        from .. import ops
        B, T, D = x.shape
        native = x.is_cuda and ops.custom_ops_enabled()
        proj = native and ops.dense_supported(x, self.wqkv.weight)
        qkv = ops.linear(x, self.wqkv.weight) if proj else self.wqkv(x)
        if native and ops.rope_split_supported(qkv, self.nh):
            # head split, RoPE and the [B, heads, T, hd] layout in one kernel
            q, k, v = ops.rope_split(qkv, cos, sin, self.nh)
        else:
            q, k, v = qkv.chunk(3, dim=-1)
            q = q.view(B, T, self.nh, self.hd).transpose(1, 2)
            k = k.view(B, T, self.nh, self.hd).transpose(1, 2)
            v = v.view(B, T, self.nh, self.hd).transpose(1, 2)
            q = _rope(q, cos, sin).to(v.dtype)
            k = _rope(k, cos, sin).to(v.dtype)
        if native and ops.attention_supported(x, self.nh):
            o = ops.attention(q, k, v, causal=True)      # tcgen05 flash attention, fwd and bwd
        else:
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        o = o.transpose(1, 2).reshape(B, T, D)
        return ops.linear(o, self.wo.weight) if proj else self.wo(o)


class Block(nn.Module):
    def __init__(self, a: ModelArgs, moe: bool):
        super().__init__()
        self.dim = a.dim
        self.n1 = nn.Parameter(torch.ones(a.dim))
        self.n2 = nn.Parameter(torch.ones(a.dim))
        self.attn = Attention(a)
        self.is_moe = moe
        if not moe:
            self.ffn = SwiGLU(a.dim, 4 * a.dim)
            return
        cfg = TRouteConfig(a.n_experts, a.n_groups, a.top_k, a.top_groups)
        if a.ep_mode != "local":
            from ..parallel.moe_layer import EPTerracedMoE
            self.ffn = EPTerracedMoE(a.dim, a.d_expert, a.d_shared, cfg, n_shared=a.n_shared,
                                     bias_gamma=a.bias_gamma, mode=a.ep_mode, rpn=a.ep_rpn,
                                     fused=a.ep_fused, capacity_factor=a.capacity_factor)
        elif a.arch == "hier":
            self.ffn = HierarchicalMoE(a.dim, a.d0, a.d1, a.p_hard, cfg, n_shared=a.n_shared,
                                       d_shared=a.d_shared, bias_gamma=a.bias_gamma)
        elif a.arch == "flat":
            self.ffn = TerracedMoE(a.dim, a.d_expert, a.d_shared, cfg, n_shared=a.n_shared,
                                   bias_gamma=a.bias_gamma, capacity_factor=a.capacity_factor)
        else:
            raise ValueError(f"unknown arch {a.arch!r}; expected 'flat' or 'hier'")
        self.ffn.routing_mode = a.routing_mode
        self.ffn.expert_backend = a.expert_backend

    def forward(self, x, cos, sin):
        x = x + self.attn(rmsnorm(x, self.n1), cos, sin)
        h = rmsnorm(x, self.n2)
        if self.is_moe:
            y, stats = self.ffn(h)
            return x + y, stats
        return x + self.ffn(h), None


class TerraceLM(nn.Module):
    def __init__(self, a: ModelArgs):
        super().__init__()
        self.args = a
        self.tok = nn.Embedding(a.vocab, a.dim)

        def is_moe(i: int) -> bool:
            if a.moe_every_layer:
                return True
            return a.dense_first <= i < a.n_layers - 1

        self.blocks = nn.ModuleList(Block(a, is_moe(i)) for i in range(a.n_layers))
        self.nf = nn.Parameter(torch.ones(a.dim))
        self.head = nn.Linear(a.dim, a.vocab, bias=False)
        hd = a.dim // a.n_heads
        inv_freq = 1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd))
        angle = torch.outer(torch.arange(a.seq_len).float(), inv_freq)
        self.register_buffer("cos", angle.cos()[None, None], persistent=False)
        self.register_buffer("sin", angle.sin()[None, None], persistent=False)

    def forward(self, idx: torch.Tensor, targets: torch.Tensor | None = None):
        T = idx.shape[1]
        if T > self.args.seq_len:
            raise ValueError(f"sequence length {T} exceeds the RoPE table ({self.args.seq_len})")
        x = self.tok(idx)
        cos, sin = self.cos[..., :T, :], self.sin[..., :T, :]
        loads, routes, gate_l, idx_l = [], [], [], []
        ep_status = None
        for blk in self.blocks:
            x, stats = blk(x, cos, sin)
            if stats is None:
                continue
            ep_status = stats.get("ep_status", ep_status)
            loads.append(stats["expert_load"])
            gate_l.append(stats["gates"])
            idx_l.append(stats["expert_idx"])
            if getattr(self, "collect_routes", False):
                routes.append(stats["expert_idx"])
        h = rmsnorm(x, self.nf)
        if targets is not None and self.args.ce_chunk > 0 and torch.is_grad_enabled():
            lm = chunked_lm_loss(h, self.head.weight, targets, self.args.ce_chunk)
        else:
            logits = self.head(h)
            if targets is None:
                return logits, {}
            lm = F.cross_entropy(logits.view(-1, logits.size(-1)).float(), targets.reshape(-1))
        if self.args.balance_aux and loads:
            aux = _balance_aux(loads, gate_l, idx_l, self.args)
        else:
            aux = lm.new_zeros(())
        loss = lm + self.args.balance_aux * aux
        info = {"lm_loss": lm.detach(), "aux": aux.detach(), "loads": loads, "routes": routes}
        if ep_status is not None:        # device status word of the fused transport (no sync)
            info["ep_status"] = ep_status
        return loss, info

    def n_params(self) -> int:
        return sum(p.numel() for p in self.parameters())


def _balance_aux(loads, gates, idxs, a: ModelArgs):
    """``E * sum_i f_i * P_i`` per MoE layer, averaged over layers.  ``f`` (share of picks per
    expert) is detached; the gradient reaches the router through ``P`` (mean gate mass)."""
    total = None
    for load, g, idx in zip(loads, gates, idxs):
        share = (load / load.sum().clamp_min(1)).detach()
        mass = torch.zeros_like(load).index_add(0, idx.reshape(-1),
                                                g.reshape(-1).to(load.dtype))
        mass = mass / max(idx.shape[0], 1)
        term = a.n_experts * (share * mass).sum()
        total = term if total is None else total + term
    return total / max(len(loads), 1)
