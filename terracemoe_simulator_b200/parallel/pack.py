"""Collective packing: several per-row planes travel as ONE int64 container per exchange.

Parity with the reference ``terrace/ta2a_pack.py``:
  * ``pack_mode`` / ``pack_enabled`` / ``reset`` (env ``TERRACE_TA2A_PACK``: unset -> ``small``;
    ``0/off/no``; ``1/small/meta``; ``full/2/all``; anything else raises)   -> ta2a_pack.py:114-175
  * ``attach_edge`` (zero-work forward, backward = reverse exchange)      -> ta2a_pack.py:212-247
  * Hop A full layout ``[id words | payload | gates | pad]``              -> ta2a_pack.py:276-358
  * Hop A small layout ``[id words | gates | pad]``                       -> ta2a_pack.py:361-423
  * ``hopa_exchange_raw`` / ``hopa_exchange_async``                       -> ta2a_pack.py:426-439
  * Hop B meta ``[slot | gate | pad]`` = 2 words per pair                 -> ta2a_pack.py:469-506
  * ``assert_not_aliased``                                                -> ta2a_pack.py:509-523

Layout rule: 8-byte id words first, then the float planes, zero padding up to a whole word.
Unpacked planes are fresh storage (never views of the container), so the container can be
freed right after unpacking.  The fused peer-memory kernels write header and payload in one
pass and need none of this; the module serves the ``torch.distributed`` arm.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .ep import CALLS, _a2a_raw, _as_list

_MODE: str | None = None
_OFF = {"0", "off", "no", "false"}
_SMALL = {"1", "small", "meta", "on", "true", "yes"}
_FULL = {"2", "full", "all"}

# live-path counters (tests prove the packed path really ran)
PACK_CALLS = {"hopa_small": 0, "hopa_full": 0, "hopb_meta": 0}


def pack_mode() -> str:
    """``off`` | ``small`` | ``full``; decided once per process from ``TERRACE_TA2A_PACK``."""
    global _MODE
    if _MODE is None:
        raw = os.environ.get("TERRACE_TA2A_PACK")
        if raw is None or raw.strip() == "":
            _MODE = "small"
        else:
            v = raw.strip().lower()
            if v in _OFF:
                _MODE = "off"
            elif v in _SMALL:
                _MODE = "small"
            elif v in _FULL:
                _MODE = "full"
            else:
                raise ValueError(f"TERRACE_TA2A_PACK={raw!r} is not a known packing mode "
                                 f"(off | small | full)")
    return _MODE


def pack_enabled() -> bool:
    return pack_mode() != "off"


def reset() -> None:
    global _MODE
    _MODE = None


def _words(nbytes: int) -> int:
    return (nbytes + 7) // 8


def _own(t: torch.Tensor) -> torch.Tensor:
    """A copy with its own storage (``contiguous`` would return a view for a dense slice)."""
    return t.clone(memory_format=torch.contiguous_format)


class _PackedEdge(torch.autograd.Function):
    """Ties a plane that was shipped inside a container back into the autograd graph: forward
    returns the already-received plane, backward sends its gradient the reverse way."""

    @staticmethod
    def forward(ctx, src, recvd, in_splits, out_splits, group):
        ctx.in_l, ctx.out_l, ctx.group = _as_list(in_splits), _as_list(out_splits), group
        return recvd.view_as(recvd)

    @staticmethod
    def backward(ctx, g):
        return _a2a_raw(g, ctx.out_l, ctx.in_l, ctx.group), None, None, None, None


def attach_edge(src, recvd, in_splits, out_splits, group):
    if src.requires_grad and torch.is_grad_enabled():
        return _PackedEdge.apply(src, recvd, in_splits, out_splits, group)
    return recvd


# ---------------------------------------------------------------------------------------------
# Hop A containers
# ---------------------------------------------------------------------------------------------
class HopASmallLayout:
    """``[id_w id words | gate_w gates of ``dtype`` | zero pad]`` per row."""
    __slots__ = ("gate_w", "id_w", "id_1d", "dtype", "gate_bytes", "words")

    def __init__(self, gate_w: int, id_w: int, id_1d: bool, dtype: torch.dtype):
        self.gate_w, self.id_w, self.id_1d, self.dtype = gate_w, id_w, id_1d, dtype
        self.gate_bytes = gate_w * torch.empty((), dtype=dtype).element_size()
        self.words = id_w + _words(self.gate_bytes)

    def __repr__(self):
        return (f"HopASmallLayout(gate_w={self.gate_w}, id_w={self.id_w}, id_1d={self.id_1d}, "
                f"dtype={self.dtype}, words={self.words})")


class HopALayout(HopASmallLayout):
    """``[id words | hidden payload elements | gates | zero pad]`` per row (payload and gates
    share one dtype)."""
    __slots__ = ("hidden", "payload_bytes")

    def __init__(self, hidden: int, gate_w: int, id_w: int, id_1d: bool, dtype: torch.dtype):
        super().__init__(gate_w, id_w, id_1d, dtype)
        self.hidden = hidden
        esz = torch.empty((), dtype=dtype).element_size()
        self.payload_bytes = hidden * esz
        self.words = id_w + _words(self.payload_bytes + self.gate_bytes)

    def __repr__(self):
        return (f"HopALayout(hidden={self.hidden}, gate_w={self.gate_w}, id_w={self.id_w}, "
                f"id_1d={self.id_1d}, dtype={self.dtype}, words={self.words})")


class PackMismatch(RuntimeError, TypeError, ValueError):
    """A plane handed to a packer has the wrong dtype, shape or row count.  It is a RuntimeError
    (what the reference raises here), and also a TypeError / ValueError for callers that tell
    the two kinds of mistake apart."""


class PackAliasError(RuntimeError, AssertionError):
    """An unpacked plane still shares storage with its container."""


def _check_ids(ids: torch.Tensor, n: int):
    if ids.dtype != torch.int64:
        raise PackMismatch(f"id plane must be int64, got {ids.dtype}")
    if ids.shape[0] != n:
        raise PackMismatch(f"id plane has {ids.shape[0]} rows, expected {n}")
    return ids.dim() == 1


def hopa_small_layout(gate_rows: torch.Tensor, ids: torch.Tensor) -> HopASmallLayout:
    id_1d = _check_ids(ids, gate_rows.shape[0])
    return HopASmallLayout(gate_rows.shape[1], 1 if id_1d else ids.shape[1], id_1d,
                           gate_rows.dtype)


def hopa_layout(payload: torch.Tensor, gate_rows: torch.Tensor, ids: torch.Tensor) -> HopALayout:
    if payload.dtype != gate_rows.dtype:
        raise PackMismatch(f"payload dtype {payload.dtype} != gate dtype {gate_rows.dtype}: the full "
                        f"container holds both planes in one dtype")
    if payload.shape[0] != gate_rows.shape[0]:
        raise PackMismatch("payload and gate planes disagree on the row count")
    id_1d = _check_ids(ids, payload.shape[0])
    return HopALayout(payload.shape[1], gate_rows.shape[1], 1 if id_1d else ids.shape[1], id_1d,
                      payload.dtype)


def hopa_pack_small(gate_rows: torch.Tensor, ids: torch.Tensor):
    lay = hopa_small_layout(gate_rows, ids)
    n = gate_rows.shape[0]
    buf = torch.zeros(n, lay.words, dtype=torch.int64, device=gate_rows.device)
    buf[:, :lay.id_w] = ids.view(n, lay.id_w)
    raw = buf.view(torch.uint8).view(n, lay.words * 8)
    raw[:, lay.id_w * 8: lay.id_w * 8 + lay.gate_bytes] = \
        gate_rows.detach().contiguous().view(torch.uint8).view(n, lay.gate_bytes)
    PACK_CALLS["hopa_small"] += 1
    return buf, lay


def hopa_unpack_small(buf: torch.Tensor, lay: HopASmallLayout):
    n = buf.shape[0]
    ids = _own(buf[:, :lay.id_w])
    if lay.id_1d:
        ids = ids.view(n)
    raw = buf.view(torch.uint8).view(n, lay.words * 8)
    gates = _own(raw[:, lay.id_w * 8: lay.id_w * 8 + lay.gate_bytes]).view(lay.dtype)
    return gates.view(n, lay.gate_w), ids


def hopa_pack(payload: torch.Tensor, gate_rows: torch.Tensor, ids: torch.Tensor):
    lay = hopa_layout(payload, gate_rows, ids)
    n = payload.shape[0]
    buf = torch.zeros(n, lay.words, dtype=torch.int64, device=payload.device)
    buf[:, :lay.id_w] = ids.view(n, lay.id_w)
    raw = buf.view(torch.uint8).view(n, lay.words * 8)
    a = lay.id_w * 8
    raw[:, a: a + lay.payload_bytes] = \
        payload.detach().contiguous().view(torch.uint8).view(n, lay.payload_bytes)
    b = a + lay.payload_bytes
    raw[:, b: b + lay.gate_bytes] = \
        gate_rows.detach().contiguous().view(torch.uint8).view(n, lay.gate_bytes)
    PACK_CALLS["hopa_full"] += 1
    return buf, lay


def hopa_unpack(buf: torch.Tensor, lay: HopALayout):
    n = buf.shape[0]
    ids = _own(buf[:, :lay.id_w])
    if lay.id_1d:
        ids = ids.view(n)
    raw = buf.view(torch.uint8).view(n, lay.words * 8)
    a = lay.id_w * 8
    payload = _own(raw[:, a: a + lay.payload_bytes]).view(lay.dtype).view(n, lay.hidden)
    b = a + lay.payload_bytes
    gates = _own(raw[:, b: b + lay.gate_bytes]).view(lay.dtype).view(n, lay.gate_w)
    return payload, gates, ids


def hopa_exchange_raw(buf, in_splits, out_splits, group=None):
    return _a2a_raw(buf, in_splits, out_splits, group)


def hopa_exchange_async(buf, in_splits, out_splits, group=None):
    """Start the container exchange; returns ``(out, work)`` -- call ``work.wait()`` before use."""
    in_l, out_l = _as_list(in_splits), _as_list(out_splits)
    out = buf.new_empty((sum(out_l), *buf.shape[1:]))
    CALLS["a2a"] += 1
    work = dist.all_to_all_single(out, buf.contiguous(), out_l, in_l, group=group, async_op=True)
    return out, work


# ---------------------------------------------------------------------------------------------
# Hop B meta container: [slot | gate | pad] = 2 words per pair
# ---------------------------------------------------------------------------------------------
def hopb_meta_words() -> int:
    return 2


def hopb_pack_meta(slot_idx: torch.Tensor, gate_pairs: torch.Tensor) -> torch.Tensor:
    if slot_idx.dtype != torch.int64:
        raise PackMismatch(f"slot plane must be int64, got {slot_idx.dtype}")
    if slot_idx.shape != gate_pairs.shape or slot_idx.dim() != 1:
        raise PackMismatch("slot and gate planes must be 1-D and of equal length")
    if not gate_pairs.is_floating_point():
        raise PackMismatch(f"gate plane must be floating point, got {gate_pairs.dtype}")
    esz = gate_pairs.element_size()
    if esz > 8:
        raise PackMismatch(f"gate dtype {gate_pairs.dtype} does not fit one word")
    n = slot_idx.shape[0]
    buf = torch.zeros(n, 2, dtype=torch.int64, device=slot_idx.device)
    buf[:, 0] = slot_idx
    raw = buf.view(torch.uint8).view(n, 16)
    raw[:, 8: 8 + esz] = gate_pairs.detach().contiguous().view(torch.uint8).view(n, esz)
    PACK_CALLS["hopb_meta"] += 1
    return buf


def hopb_unpack_meta(buf: torch.Tensor, dtype: torch.dtype):
    n = buf.shape[0]
    esz = torch.empty((), dtype=dtype).element_size()
    slot = _own(buf[:, 0])
    raw = buf.view(torch.uint8).view(n, 16)
    gate = _own(raw[:, 8: 8 + esz]).view(dtype).view(n)
    return slot, gate


def assert_not_aliased(buf: torch.Tensor, *planes: torch.Tensor) -> None:
    """Trip if an unpacked plane still shares storage with the container it came from."""
    if buf.numel() == 0:
        return
    base = buf.untyped_storage().data_ptr()
    for i, p in enumerate(planes):
        if p.numel() and p.untyped_storage().data_ptr() == base:
            raise PackAliasError(f"unpacked plane #{i} aliases its container (shared storage); "
                                 f"freeing the container would invalidate it")
