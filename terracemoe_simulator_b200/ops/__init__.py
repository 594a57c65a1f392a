"""Native-op loader, gate and autograd wrappers.

Parity with the reference ``terrace/ops/__init__.py``:
  * tri-state gate from ``TERRACE_CUSTOM_OPS`` (``0`` off, ``1`` try and fall back with ONE
    warning, ``require``/``2`` raise), explicit library path ``TERRACE_OPS_LIB``, default
    search ``ops/lib/*.so``, all-or-nothing required op set, decided once and cached
    (``OpsState``)                                                -> ops/__init__.py:53-190
  * ``passthrough`` / ``TerracePassthroughFn``                    -> ops/__init__.py:197-242
  * ``k1_arrival_ref``, adjoints, ``TerraceK1ArrivalFn``, ``k1_arrival``, two-edge
    ``k1_arrival_segment``                                        -> ops/__init__.py:255-474
  * ``k2_pack`` dispatcher over ``k2_pack_ref``                   -> ops/k2_ref.py

One deliberate difference: with the variable UNSET the reference stays off; here an unset
variable means ``auto`` -- off on a machine without CUDA, ``require`` on a machine with a
GPU, so that a GPU box never falls back to eager silently when the extension is missing.
"""
from __future__ import annotations

import glob
import logging
import os
from dataclasses import dataclass

import torch

from .refs import fixed_hist, k1_arrival_ref, k2_pack_ref, stable_bucket_order

log = logging.getLogger("terrace.ops")

_LIB_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib")
_REQUIRED_OPS = ("passthrough", "k1_arrival", "k2_pack")
NAMESPACE = "terrace"

# live-path counters
OP_CALLS: dict = {}


def _count(name: str) -> None:
    OP_CALLS[name] = OP_CALLS.get(name, 0) + 1


class OpsLoadError(RuntimeError):
    pass


@dataclass(frozen=True)
class OpsState:
    requested: str          # "0" | "1" | "require"
    loaded: bool
    lib: str | None
    reason: str


_STATE: OpsState | None = None


def _normalized_switch() -> str:
    raw = os.environ.get("TERRACE_CUSTOM_OPS")
    if raw is None or raw.strip() == "":
        return "require" if torch.cuda.is_available() else "0"
    v = raw.strip().lower()
    if v in ("0", "off", "false", "no"):
        return "0"
    if v in ("1", "on", "true", "yes", "try"):
        return "1"
    if v in ("2", "require", "required"):
        return "require"
    raise ValueError(f"TERRACE_CUSTOM_OPS={raw!r} is not understood (0 | 1 | require)")


def _find_library() -> str | None:
    explicit = os.environ.get("TERRACE_OPS_LIB")
    if explicit:
        return explicit if os.path.isfile(explicit) else None
    hits = sorted(glob.glob(os.path.join(_LIB_DIR, "terrace_b200_ops*.so")))
    return hits[0] if hits else None


def _try_load() -> tuple[bool, str | None, str]:
    lib = _find_library()
    if lib is None:
        return False, None, (f"no native library found (TERRACE_OPS_LIB unset or missing, "
                             f"nothing under {_LIB_DIR}); build it with "
                             f"`python -m terracemoe_simulator_b200.ops.build`")
    from ..utils.flags import check_native_flags
    check_native_flags()      # the GEMM policy switches are read by C++: unknown values raise here
    try:
        torch.ops.load_library(lib)
    except Exception as exc:  # noqa: BLE001 - any loader failure is reported the same way
        return False, lib, f"loading {lib} failed: {exc!r}"
    ns = getattr(torch.ops, NAMESPACE)
    missing = [op for op in _REQUIRED_OPS if not hasattr(ns, op)]
    if missing:
        return False, lib, f"{lib} lacks required ops {missing}"
    return True, lib, "loaded"


def _initialize() -> OpsState:
    switch = _normalized_switch()
    if switch == "0":
        raw = os.environ.get("TERRACE_CUSTOM_OPS")
        why = "explicit off (TERRACE_CUSTOM_OPS=0)" if raw not in (None, "") else \
            "native ops off by default on a host without CUDA"
        return OpsState("0", False, None, why)
    ok, lib, reason = _try_load()
    if ok:
        log.info("terrace native ops loaded from %s", lib)
        return OpsState(switch, True, lib, reason)
    if switch == "require":
        raise OpsLoadError(f"TERRACE_CUSTOM_OPS requires the native ops but {reason}")
    log.warning("terrace native ops unavailable, falling back to PyTorch ops: %s", reason)
    return OpsState(switch, False, lib, reason)


def status() -> OpsState:
    global _STATE
    if _STATE is None:
        _STATE = _initialize()
    return _STATE


def custom_ops_enabled() -> bool:
    return status().loaded


def reset() -> None:
    """Forget the cached decision (test hook)."""
    global _STATE
    _STATE = None


def _ns():
    return getattr(torch.ops, NAMESPACE)


# ---------------------------------------------------------------------------------------------
# passthrough (toolchain + loader smoke op)
# ---------------------------------------------------------------------------------------------
class TerracePassthroughFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        _count("passthrough")
        return _ns().passthrough(x)

    @staticmethod
    def backward(ctx, g):
        return g


def passthrough(x: torch.Tensor) -> torch.Tensor:
    """``y = x`` as a fresh tensor: the identity kernel when native ops are on, else a clone."""
    if custom_ops_enabled() and x.is_cuda:
        return TerracePassthroughFn.apply(x)
    return x.clone()


# ---------------------------------------------------------------------------------------------
# K1: arrival chain
# ---------------------------------------------------------------------------------------------
def _k1_grad_rx(g_send: torch.Tensor, r_idx: torch.Tensor, rx_shape) -> torch.Tensor:
    """Adjoint of ``send_buf = rx[r_idx]``: pair gradients added per row in pair order (slot
    ascending), accumulated in fp32 and rounded once."""
    acc = torch.zeros(rx_shape, dtype=torch.float32, device=g_send.device)
    acc.index_add_(0, r_idx, g_send.float())
    return acc.to(g_send.dtype)


def _k1_grad_rgate(g_gate: torch.Tensor, rslot: torch.Tensor, epr: int, rpn: int, rgate_shape):
    """Adjoint of ``gate_pairs = rgate.flatten()[order]`` (a permutation: no reduction)."""
    order = stable_bucket_order(torch.div(rslot.reshape(-1), epr, rounding_mode="floor"), rpn)
    flat = g_gate.new_zeros(rgate_shape[0] * rgate_shape[1])
    flat.index_copy_(0, order, g_gate)
    return flat.view(rgate_shape)


def _k1_forward(rx, rslot, rgate, quota, epr, rpn, my_local):
    if custom_ops_enabled() and rx.is_cuda and rgate.dtype == rx.dtype:
        _count("k1_arrival")
        return _ns().k1_arrival(rx, rslot, rgate, quota, epr, rpn, my_local)
    return k1_arrival_ref(rx, rslot, rgate, quota, epr, rpn, my_local)


class TerraceK1ArrivalFn(torch.autograd.Function):
    """Fused arrival node: native forward, composed-chain backward."""

    @staticmethod
    def forward(ctx, rx, rslot, rgate, quota, epr, rpn, my_local):
        out = _k1_forward(rx, rslot, rgate, quota, epr, rpn, my_local)
        send_buf, gate_pairs, r_idx, slot_idx, i_send = out
        ctx.save_for_backward(r_idx, rslot)
        ctx.geom = (epr, rpn, tuple(rx.shape), tuple(rgate.shape))
        ctx.mark_non_differentiable(r_idx, slot_idx, i_send)
        return send_buf, gate_pairs, r_idx, slot_idx, i_send

    @staticmethod
    def backward(ctx, g_send, g_gate, *_):
        r_idx, rslot = ctx.saved_tensors
        epr, rpn, rx_shape, rgate_shape = ctx.geom
        g_rx = _k1_grad_rx(g_send.contiguous(), r_idx, rx_shape) if g_send is not None else None
        g_rg = (_k1_grad_rgate(g_gate.contiguous(), rslot, epr, rpn, rgate_shape)
                if g_gate is not None else None)
        return g_rx, None, g_rg, None, None, None, None


def k1_arrival(rx, rslot, rgate, quota: int, epr: int, rpn: int, my_local: int = 0):
    """Arrival chain with gradients to ``rx`` and ``rgate`` (native kernel when enabled)."""
    if rx.dim() != 2 or rslot.dim() != 2 or rgate.shape != rslot.shape:
        raise ValueError("k1_arrival: rx must be [R,H]; rslot and rgate [R,q]")
    if rslot.dtype != torch.int64:
        raise TypeError("k1_arrival: rslot must be int64")
    if not 0 <= my_local < rpn:
        raise ValueError(f"k1_arrival: my_local={my_local} outside [0, {rpn})")
    return TerraceK1ArrivalFn.apply(rx, rslot, rgate, quota, epr, rpn, my_local)


class _K1SendEdge(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rx, send_buf, r_idx):
        ctx.save_for_backward(r_idx)
        ctx.shape = tuple(rx.shape)
        return send_buf.view_as(send_buf)

    @staticmethod
    def backward(ctx, g):
        (r_idx,) = ctx.saved_tensors
        return _k1_grad_rx(g.contiguous(), r_idx, ctx.shape), None, None


class _K1GateEdge(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rgate, gate_pairs, rslot, epr, rpn):
        ctx.save_for_backward(rslot)
        ctx.geom = (epr, rpn, tuple(rgate.shape))
        return gate_pairs.view_as(gate_pairs)

    @staticmethod
    def backward(ctx, g):
        (rslot,) = ctx.saved_tensors
        epr, rpn, shape = ctx.geom
        return _k1_grad_rgate(g.contiguous(), rslot, epr, rpn, shape), None, None, None, None


def k1_arrival_segment(rx, rslot, rgate, quota: int, epr: int, rpn: int, my_local: int = 0):
    """Same five outputs as :func:`k1_arrival`, but ``send_buf`` and ``gate_pairs`` hang on two
    DISJOINT autograd edges, for callers that run two separate ``backward`` calls (one through
    the payload, one through the gate)."""
    with torch.no_grad():
        send_buf, gate_pairs, r_idx, slot_idx, i_send = _k1_forward(
            rx, rslot, rgate, quota, epr, rpn, my_local)
    if torch.is_grad_enabled():
        if rx.requires_grad:
            send_buf = _K1SendEdge.apply(rx, send_buf, r_idx)
        if rgate.requires_grad:
            gate_pairs = _K1GateEdge.apply(rgate, gate_pairs, rslot, epr, rpn)
    return send_buf, gate_pairs, r_idx, slot_idx, i_send


# ---------------------------------------------------------------------------------------------
# K2: send-side pack
# ---------------------------------------------------------------------------------------------
class TerraceK2PackFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, expert_idx, gates, world, n_experts, rpn, groups_m):
        if custom_ops_enabled() and hidden.is_cuda:
            _count("k2_pack")
            out = _ns().k2_pack(hidden, expert_idx, gates, world, n_experts, rpn, groups_m)
        else:
            out = k2_pack_ref(hidden, expert_idx, gates, world, n_experts, rpn, groups_m)
        payload, mask, gate_rows, u_src, node_counts = out
        ctx.save_for_backward(u_src, expert_idx)
        ctx.geom = (tuple(hidden.shape), world, n_experts, rpn, groups_m)
        ctx.mark_non_differentiable(mask, u_src, node_counts)
        return payload, mask, gate_rows, u_src, node_counts

    @staticmethod
    def backward(ctx, g_payload, _gm, g_gate_rows, *_):
        u_src, expert_idx = ctx.saved_tensors
        shape, world, n_experts, rpn, m = ctx.geom
        g_hidden = g_gates = None
        if g_payload is not None:
            acc = torch.zeros(shape, dtype=torch.float32, device=g_payload.device)
            acc.index_add_(0, u_src, g_payload.float())          # row order = group ascending
            g_hidden = acc.to(g_payload.dtype)
        if g_gate_rows is not None:
            T, k = expert_idx.shape
            q = k // m
            slots = (n_experts // world) * rpn
            e_sorted, cols = torch.sort(expert_idx, dim=1, stable=True)
            dest = torch.div(e_sorted[:, ::q], slots, rounding_mode="floor").reshape(-1)
            order = stable_bucket_order(dest, world // rpn)
            sorted_g = g_gate_rows.new_zeros(T * m, q)
            sorted_g.index_copy_(0, order, g_gate_rows)
            g_gates = torch.zeros_like(sorted_g.view(T, k)).scatter_(1, cols, sorted_g.view(T, k))
        return g_hidden, None, g_gates, None, None, None, None


def k2_pack(hidden, expert_idx, gates, world: int, n_experts: int, rpn: int, groups_m: int):
    """Send-side pack with gradients to ``hidden`` and ``gates``."""
    return TerraceK2PackFn.apply(hidden, expert_idx, gates, world, n_experts, rpn, groups_m)


# ---------------------------------------------------------------------------------------------
# compute kernels (wrappers live in native.py; they import lazily so CPU-only use stays light)
# ---------------------------------------------------------------------------------------------
from .native import (  # noqa: E402
    attention, attention_shape_supported, attention_supported, dense_supported, fused_route, grouped_mm_native,
    grouped_supported, linear, moe_experts_local, moe_local_supported, rmsnorm, rmsnorm_supported,
    rope_split, rope_split_supported, route_from_logits, route_fused_supported, route_hidden,
    router_supported,
    segments_from_counts, swiglu_ffn, take_status)

__all__ = [
    "OpsLoadError", "OpsState", "status", "custom_ops_enabled", "reset", "passthrough",
    "TerracePassthroughFn", "k1_arrival", "k1_arrival_ref", "k1_arrival_segment",
    "TerraceK1ArrivalFn", "k2_pack", "k2_pack_ref", "fixed_hist", "stable_bucket_order",
    "rmsnorm", "fused_route", "linear", "swiglu_ffn", "grouped_mm_native", "moe_experts_local",
    "attention", "OP_CALLS",
]
