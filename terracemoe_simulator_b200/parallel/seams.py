"""Split seams of the T-A2A dispatch for MoE layers that own their expert computation.

``ta2a_permute`` does everything up to the expert GEMM input (plan, Hop A, arrival chain, Hop B,
sort by local expert) and returns ``(permuted_rows, tokens_per_expert, permuted_probs, state)``;
the caller multiplies its expert outputs by ``permuted_probs`` and hands them to
``ta2a_unpermute``, which runs the return leg WITHOUT gates (they were applied by the caller).
Unlike the closed forward (``parallel/ta2a.py``), the gate therefore rides Hop B to the expert
rank.

Parity with the reference ``terrace/ta2a_dispatch.py``:
  * ``TA2AState``                                   -> ta2a_dispatch.py:62-74
  * env gates (async counts, early Hop B counts, sync probe, shared overlap, ``ta2a_enabled``)
                                                    -> ta2a_dispatch.py:102-178, 614-639, 1016-1020
  * ``routing_map_to_topk``                         -> ta2a_dispatch.py:224-260
  * ``ta2a_permute`` / ``ta2a_unpermute``           -> ta2a_dispatch.py:263-498
  * overlap variants (async Hop A under a shared-expert callback, ``save_tensors`` seats)
                                                    -> ta2a_dispatch.py:655-1013
The overlap variants here keep the call signature and the seat layout (7 tensors appended by
the permute, 3 by the un-permute) but rely on regular autograd instead of a vendor-driven manual
backward replay; their results are bit-identical to the plain seams.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .. import ops
from ..ops.refs import fixed_hist, stable_bucket_order
from ..utils import drift_probe as _dp
from . import pack as _pack
from .ep import CALLS, _a2a, _a2a_raw
from .plan import plan_ta2a
from .ta2a import _RowGather, build_expansion, expand_arrival_mask, pack_quota_wire

_FLAGS: dict = {}
SEAM_CALLS = {"permute": 0, "unpermute": 0, "permute_overlap": 0, "unpermute_overlap": 0,
              "async_counts": 0, "early_hopb": 0, "sync_probe": 0}


def _env_flag(name: str, default: bool) -> bool:
    if name not in _FLAGS:
        raw = os.environ.get(name)
        if raw is None or raw.strip() == "":
            _FLAGS[name] = default
        else:
            v = raw.strip().lower()
            if v in ("1", "on", "true", "yes"):
                _FLAGS[name] = True
            elif v in ("0", "off", "false", "no"):
                _FLAGS[name] = False
            else:
                raise ValueError(f"{name}={raw!r} is not a boolean switch (0 | 1)")
    return _FLAGS[name]


def async_counts_enabled() -> bool:
    return _env_flag("TERRACE_TA2A_ASYNC_COUNTS", True)


def early_hopb_counts_enabled() -> bool:
    return _env_flag("TERRACE_TA2A_EARLY_HOPB", True)


def sync_probe_enabled() -> bool:
    return _env_flag("TERRACE_TA2A_SYNC_PROBE", False)


def shared_overlap_enabled() -> bool:
    return _env_flag("TERRACE_SHARED_OVERLAP", True)


def reset_async_counts() -> None:
    _FLAGS.pop("TERRACE_TA2A_ASYNC_COUNTS", None)


def reset_early_hopb() -> None:
    _FLAGS.pop("TERRACE_TA2A_EARLY_HOPB", None)


def reset_sync_probe() -> None:
    _FLAGS.pop("TERRACE_TA2A_SYNC_PROBE", None)


def reset_shared_overlap() -> None:
    _FLAGS.pop("TERRACE_SHARED_OVERLAP", None)


def ta2a_enabled(ep_world: int, rpn: int = 8) -> bool:
    """T-A2A applies when ``TERRACE_TA2A=1`` and the EP world spans at least two groups."""
    raw = os.environ.get("TERRACE_TA2A", "").strip().lower()
    return raw in ("1", "on", "true", "yes") and ep_world // max(rpn, 1) >= 2


class TA2AState:
    __slots__ = ("u_src", "r_idx", "order", "R", "T", "hidden", "send_l", "recv_l", "is_l",
                 "ir_l", "intra", "inter", "dtype")

    def __init__(self, **kw):
        for name in self.__slots__:
            setattr(self, name, kw.get(name))


def routing_map_to_topk(routing_map: torch.Tensor, probs: torch.Tensor):
    """Dense ``routing_map[T, E]`` (bool) + ``probs[T, E]`` -> ascending ``expert_idx[T, k]`` and
    the matching ``gates[T, k]``.  One host sync (to read k); raises unless every row selects
    exactly the same number of experts."""
    if routing_map.shape != probs.shape or routing_map.dim() != 2:
        raise ValueError("routing_map and probs must both be [T, E]")
    per_row = routing_map.sum(dim=1)
    T = routing_map.shape[0]
    if T == 0:
        return routing_map.new_zeros((0, 0), dtype=torch.int64), probs.new_zeros((0, 0))
    lo, hi = int(per_row.min()), int(per_row.max())
    if lo != hi:
        raise ValueError(f"routing_map must select exactly k experts per token; rows select "
                         f"between {lo} and {hi}")
    k = lo
    expert_idx = routing_map.nonzero(as_tuple=False)[:, 1].view(T, k)   # row-major: ascending
    return expert_idx, probs.gather(1, expert_idx)


def _group_size(group) -> int:
    return dist.get_world_size(group) if group is not None else dist.get_world_size()


def _hopa_counts(world: int, n_nodes: int, rpn: int, my_local: int, counts: torch.Tensor,
                 inter_group):
    """Per-destination Hop A send counts in the layout of the communicator that carries Hop A:
    length N_g on the inter-group sub-communicator, else length W with N_g non-zeros."""
    if inter_group is not None and _group_size(inter_group) == n_nodes:
        return counts.clone()
    send = torch.zeros(world, dtype=torch.int64, device=counts.device)
    send[torch.arange(n_nodes, device=counts.device) * rpn + my_local] = counts
    return send


def _exchange_counts(send, group, want_async: bool):
    recv = torch.empty_like(send)
    CALLS["a2a"] += 1
    if want_async:
        return recv, dist.all_to_all_single(recv, send, group=group, async_op=True)
    dist.all_to_all_single(recv, send, group=group)
    return recv, None


def _permute_core(hidden_states, probs, routing_map, *, world, rank, rpn, n_experts, intra_group,
                  inter_group, groups_m, overlap_cb=None, staged=False):
    """Shared body of the two permute seams.  ``staged`` (the overlap seam) cuts the autograd graph
    at Hop A: the payload and gate planes cross detached, outside autograd, and come back as the
    leaves ``rx_d`` / ``rgate_d`` of a second graph; the caller replays the backward segment by
    segment and moves the gradients across Hop A itself."""
    n_nodes = world // rpn
    if n_nodes < 2:
        raise ValueError("ta2a_permute needs at least two groups (world // rpn >= 2)")
    my_local = rank % rpn
    epr = n_experts // world
    slots = epr * rpn
    x = hidden_states.reshape(-1, hidden_states.shape[-1])
    T, H = x.shape
    expert_idx, gates = routing_map_to_topk(routing_map, probs)
    # the gate plane travels in the payload dtype (router-precision probabilities are rounded
    # once, here, in both seams)
    gates = gates.to(x.dtype)
    k = expert_idx.shape[1]
    u_src, u_node, counts, inverse = plan_ta2a(expert_idx, world, n_experts, rpn, groups_m)
    n_rows = u_src.shape[0]
    hop_group = inter_group if (inter_group is not None
                                and _group_size(inter_group) == n_nodes) else None
    send = _hopa_counts(world, n_nodes, rpn, my_local, counts, inter_group)
    use_async = async_counts_enabled()
    recv, work = _exchange_counts(send, hop_group, use_async)
    if use_async:
        SEAM_CALLS["async_counts"] += 1
    payload = _RowGather.apply(x, u_src)
    if groups_m is not None:
        q = k // groups_m
        ids, gate_tab, _ = pack_quota_wire(expert_idx, gates, inverse, n_rows, slots, q)
    else:
        q = None
        slot_flat = (expert_idx % slots).reshape(-1)
        ids = build_expansion(expert_idx, inverse, n_rows, world, n_experts, rpn,
                              slot_flat=slot_flat)
        gate_tab = gates.new_zeros(n_rows, slots).index_put((inverse, slot_flat),
                                                            gates.reshape(-1))
    _dp.note("seam.payload", payload)
    _dp.note("seam.gate", gate_tab)
    _dp.note_int("seam.mask", ids)
    if work is not None:
        work.wait()
    if sync_probe_enabled():
        SEAM_CALLS["sync_probe"] += 1
        _ = recv.tolist()                      # discarded read: measures the sync cost only
    send_l, recv_l = send.tolist(), recv.tolist()

    shared_out = None
    # the public switch first (callers and tests may override it), then the container form
    mode = _pack.pack_mode() if _pack.pack_enabled() else "off"
    stage1 = None
    if staged:
        # Hop A outside autograd, the payload in flight while the shared experts compute
        if shared_overlap_enabled():
            rx_buf, rx_work = _pack.hopa_exchange_async(payload.detach(), send_l, recv_l, hop_group)
            if overlap_cb is not None:
                shared_out = overlap_cb()
            rx_work.wait()
        else:
            if overlap_cb is not None:
                shared_out = overlap_cb()      # serial control arm
            rx_buf = _a2a_raw(payload.detach(), send_l, recv_l, hop_group)
        if mode in ("small", "full"):
            buf, lay = _pack.hopa_pack_small(gate_tab.detach(), ids)
            rbuf = _pack.hopa_exchange_raw(buf, send_l, recv_l, hop_group)
            rgate_raw, rids = _pack.hopa_unpack_small(rbuf, lay)
        else:
            rids = _a2a_raw(ids, send_l, recv_l, hop_group)
            rgate_raw = _a2a_raw(gate_tab.detach(), send_l, recv_l, hop_group)
        rx = rx_buf.detach().requires_grad_(True)
        rgate = rgate_raw.detach().requires_grad_(True)
        stage1 = (payload, gate_tab, rx, rgate)
        mode_payload_done = True
    elif overlap_cb is not None and shared_overlap_enabled():
        # Hop A payload in flight while the shared experts compute
        rx_buf, rx_work = _pack.hopa_exchange_async(payload.detach(), send_l, recv_l, hop_group)
        shared_out = overlap_cb()
        rx_work.wait()
        rx = _pack.attach_edge(payload, rx_buf, send_l, recv_l, hop_group)
        mode_payload_done = True
    else:
        if overlap_cb is not None:
            shared_out = overlap_cb()          # serial control arm
        mode_payload_done = False
        rx = None

    if staged:
        pass
    elif mode == "full" and not mode_payload_done and gate_tab.dtype == payload.dtype:
        buf, lay = _pack.hopa_pack(payload, gate_tab, ids)
        rbuf = _pack.hopa_exchange_raw(buf, send_l, recv_l, hop_group)
        rx_raw, rgate_raw, rids = _pack.hopa_unpack(rbuf, lay)
        rx = _pack.attach_edge(payload, rx_raw, send_l, recv_l, hop_group)
        rgate = _pack.attach_edge(gate_tab, rgate_raw, send_l, recv_l, hop_group)
    elif mode in ("small", "full"):
        buf, lay = _pack.hopa_pack_small(gate_tab, ids)
        rbuf = _pack.hopa_exchange_raw(buf, send_l, recv_l, hop_group)
        rgate_raw, rids = _pack.hopa_unpack_small(rbuf, lay)
        rgate = _pack.attach_edge(gate_tab, rgate_raw, send_l, recv_l, hop_group)
        if rx is None:
            rx = _a2a(payload, send_l, recv_l, hop_group)
    else:
        if rx is None:
            rx = _a2a(payload, send_l, recv_l, hop_group)
        rids = _a2a_raw(ids, send_l, recv_l, hop_group)
        rgate = _a2a(gate_tab, send_l, recv_l, hop_group)
    _dp.note("seam.rx", rx)
    _dp.note("seam.rgate", rgate)
    _dp.note_int("seam.rmask", rids)

    # ---- arrival chain
    R = rx.shape[0]
    if q is not None and staged:
        # the row path and the gate path must be separate graphs: the layer calls backward on
        # each of them in turn (the segment variant hangs them on two disjoint autograd edges)
        send_buf, gate_pairs, r_idx, slot_idx, i_send = ops.k1_arrival_segment(
            rx, rids.view(R, q), rgate, q, epr, rpn, my_local)
    elif q is not None:
        send_buf, gate_pairs, r_idx, slot_idx, i_send = ops.k1_arrival(
            rx, rids.view(R, q), rgate, q, epr, rpn, my_local)
    else:
        r0, s0 = expand_arrival_mask(rids.view(R), slots)
        owner = torch.div(s0, epr, rounding_mode="floor")
        order_pairs = stable_bucket_order(owner, rpn)
        r_idx, slot_idx = r0[order_pairs], s0[order_pairs]
        i_send = fixed_hist(owner, rpn)
        send_buf = _RowGather.apply(rx, r_idx)
        gate_pairs = rgate[r_idx, slot_idx]
    early = early_hopb_counts_enabled()
    i_recv, hb_work = _exchange_counts(i_send, intra_group, early)
    if early:
        SEAM_CALLS["early_hopb"] += 1
    _dp.note("seam.exprx", send_buf)
    _dp.note("seam.gpairs", gate_pairs)
    _dp.note_int("seam.slot", slot_idx)
    _dp.note_int("seam.isend", i_send)
    if hb_work is not None:
        hb_work.wait()
    is_l, ir_l = i_send.tolist(), i_recv.tolist()

    # ---- Hop B (the gate travels too: the caller applies it)
    node_rx = _a2a(send_buf, is_l, ir_l, intra_group)
    if mode != "off":
        meta = _pack.hopb_pack_meta(slot_idx, gate_pairs)
        rmeta = _a2a_raw(meta, is_l, ir_l, intra_group)
        my_slot, gate_raw = _pack.hopb_unpack_meta(rmeta, gate_pairs.dtype)
        my_gate = _pack.attach_edge(gate_pairs, gate_raw, is_l, ir_l, intra_group)
    else:
        my_slot = _a2a_raw(slot_idx, is_l, ir_l, intra_group)
        my_gate = _a2a(gate_pairs, is_l, ir_l, intra_group)
    exp_j = my_slot - my_local * epr
    order = torch.argsort(exp_j, stable=True)
    tokens_per_expert = fixed_hist(exp_j, epr)
    permuted, pprobs = node_rx[order], my_gate[order]
    _dp.note("seam.permuted", permuted)
    _dp.note("seam.pprobs", pprobs)
    _dp.note_int("seam.tpe", tokens_per_expert)
    st = TA2AState(u_src=u_src, r_idx=r_idx, order=order, R=R, T=T, hidden=H, send_l=send_l,
                   recv_l=recv_l, is_l=is_l, ir_l=ir_l, intra=intra_group, inter=hop_group,
                   dtype=x.dtype)
    if staged:
        return permuted, tokens_per_expert, pprobs, shared_out, st, stage1
    return permuted, tokens_per_expert, pprobs, shared_out, st


def ta2a_permute(hidden_states, probs, routing_map, *, world, rank, rpn, n_experts, intra_group,
                 inter_group=None, groups_m=None):
    SEAM_CALLS["permute"] += 1
    _dp.tick_dispatch()
    permuted, tpe, pprobs, _shared, st = _permute_core(
        hidden_states, probs, routing_map, world=world, rank=rank, rpn=rpn, n_experts=n_experts,
        intra_group=intra_group, inter_group=inter_group, groups_m=groups_m)
    return permuted, tpe, pprobs, st


def _unpermute_core(expert_out, st: TA2AState):
    _dp.note("seam.eout", expert_out)
    unsort = torch.empty_like(st.order)
    unsort[st.order] = torch.arange(st.order.numel(), device=st.order.device)
    ret = _a2a(expert_out[unsort], st.ir_l, st.is_l, st.intra)
    _dp.note("seam.ret", ret)
    red = torch.zeros(st.R, st.hidden, dtype=torch.float32, device=ret.device).index_add(
        0, st.r_idx, ret.float()).to(ret.dtype)
    _dp.note("seam.red", red)
    back = _a2a(red, st.recv_l, st.send_l, st.inter)
    _dp.note("seam.back", back)
    y = torch.zeros(st.T, st.hidden, dtype=torch.float32, device=back.device).index_add(
        0, st.u_src, back.float()).to(back.dtype)
    _dp.note("seam.y", y)
    return y


def ta2a_unpermute(expert_out, st: TA2AState, out_like):
    """Return leg without gates; result has ``out_like``'s shape."""
    SEAM_CALLS["unpermute"] += 1
    return _unpermute_core(expert_out, st).view(out_like.shape)


def ta2a_permute_overlap(hidden_states, probs, routing_map, *, world, rank, rpn, n_experts,
                         intra_group, inter_group=None, groups_m=None, save_tensors,
                         run_shared_experts=None):
    """Overlap seam, forward half, for a layer that replays its backward by hand.

    Hop A runs outside autograd (asynchronously, with ``run_shared_experts()`` computing while
    the payload is in flight) and the graph is cut there.  Seven entries are appended to
    ``save_tensors`` at fixed positions (``ta2a_dispatch.py:750-751, 951-955`` in the reference):

    0. the Hop A payload ``hidden[u_src]`` with its graph (stage 1),
    1. the gate plane as shipped, with its graph (stage 1),
    2. ``None`` (the seat of a host-side count tensor this implementation does not need),
    3. ``rx_d``: the received rows as a detached leaf (input of stage 2),
    4. ``permuted`` with the stage-2 graph (arrival step, Hop B, expert sort),
    5. ``rgate_d``: the received gates as a detached leaf,
    6. ``permuted_probs`` with the stage-2 graph.

    The backward of the layer calls ``permuted.backward(d_permuted)`` and
    ``permuted_probs.backward(d_probs)``, sends ``rx_d.grad`` / ``rgate_d.grad`` back over Hop A with
    ``_a2a_raw(grad, st.recv_l, st.send_l)`` and finishes with
    ``torch.autograd.backward([payload, gates], [d_payload, d_gates])``.
    Returns ``(permuted, tokens_per_expert, permuted_probs, shared_out, state)``."""
    SEAM_CALLS["permute_overlap"] += 1
    _dp.tick_dispatch()
    with torch.enable_grad():
        permuted, tpe, pprobs, shared_out, st, stage1 = _permute_core(
            hidden_states, probs, routing_map, world=world, rank=rank, rpn=rpn,
            n_experts=n_experts, intra_group=intra_group, inter_group=inter_group,
            groups_m=groups_m, overlap_cb=run_shared_experts, staged=True)
    payload, gate_tab, rx_d, rgate_d = stage1
    save_tensors.extend([payload, gate_tab, None, rx_d, permuted, rgate_d, pprobs])
    return permuted, tpe, pprobs, shared_out, st


def ta2a_unpermute_overlap(expert_out, st: TA2AState, save_tensors, out_shape=None):
    """Overlap seam, return half.  Appends three entries (``ta2a_dispatch.py:995-996, 1011``):

    7. ``eo_d``: the expert output as a detached leaf,
    8. ``red``: per-(token, group) sums at the representative, with the graph from ``eo_d``
       (un-sort, Hop B reverse, reduction over the arrival pairs),
    9. ``back_d``: the rows returned over Hop A (outside autograd) as a detached leaf, from which
       the result ``y`` is built.

    Backward by hand: ``y.backward(dy)``; ``d_red = _a2a_raw(back_d.grad, st.send_l, st.recv_l)``;
    ``red.backward(d_red)``; ``eo_d.grad`` is the gradient of the expert output."""
    SEAM_CALLS["unpermute_overlap"] += 1
    with torch.enable_grad():
        eo_d = expert_out.detach().requires_grad_(True)
        _dp.note("seam.eout", eo_d)
        unsort = torch.empty_like(st.order)
        unsort[st.order] = torch.arange(st.order.numel(), device=st.order.device)
        ret = _a2a(eo_d[unsort], st.ir_l, st.is_l, st.intra)
        red = torch.zeros(st.R, st.hidden, dtype=torch.float32, device=ret.device).index_add(
            0, st.r_idx, ret.float()).to(ret.dtype)
        _dp.note("seam.red", red)
        back = _a2a_raw(red.detach(), st.recv_l, st.send_l, st.inter)
        back_d = back.detach().requires_grad_(True)
        y = torch.zeros(st.T, st.hidden, dtype=torch.float32, device=back.device).index_add(
            0, st.u_src, back_d.float()).to(back.dtype)
        _dp.note("seam.y", y)
    save_tensors.extend([eo_d, red, back_d])
    return y.view(out_shape) if out_shape is not None else y
