"""Autograd wrappers around the sm_100a compute kernels (filled in kernel by kernel)."""
from __future__ import annotations

import torch


def _lib():
    from . import _ns
    return _ns()


def rmsnorm_supported(x, w) -> bool:
    return False


def router_supported(cfg, hidden) -> bool:
    return False


def dense_supported(x, w) -> bool:
    return False


def grouped_supported(x, w) -> bool:
    return False


def attention_supported(x, n_heads) -> bool:
    return False


def rmsnorm(x, w, eps=1e-5):
    raise NotImplementedError


def fused_route(hidden, weight, bias, cfg):
    raise NotImplementedError


def linear(x, w):
    raise NotImplementedError


def swiglu_ffn(x, w13, w2):
    raise NotImplementedError


def grouped_mm_native(x, w, counts):
    raise NotImplementedError


def moe_experts_local(x, expert_idx, gates, w13, w2):
    raise NotImplementedError


def causal_attention_rope(qkv, cos, sin):
    raise NotImplementedError
