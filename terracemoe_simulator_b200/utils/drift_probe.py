"""Drift probe: permutation-invariant fingerprints of tensors at named points of the dispatch,
for finding the FIRST place where two runs (two paths, two machines, two builds) diverge.

Switched by environment variables, read once:
  ``TERRACE_DRIFT_PROBE=1``        enable
  ``TERRACE_DRIFT_PROBE_EVERY=n``  probe every n-th dispatch (default 1)
  ``TERRACE_DRIFT_PROBE_MAXCALL``  stop after that many dispatches (default unlimited)
  ``TERRACE_DRIFT_PROBE_RANKS``    comma list of ranks that emit (default all)
  ``TERRACE_DRIFT_PROBE_STRICT=1`` contract violations raise ``DriftProbeMismatch``
  ``TERRACE_DRIFT_PROBE_CHUNK``    elements per partial sum of the float digest (default 1<<16)

A float fingerprint is ``(numel, sum|x|, sum x^2, max|x|)`` accumulated in float64 over fixed
chunks (so it does not depend on the device's reduction order); an integer fingerprint is the
exact ``(numel, sum, min, max)``.  Lines look like
``[terrace-drift] pt=seam.rx step=3 layer=7 call=12 rank=0 dt=bfloat16 n=.. sabs=.. ssq=.. amax=..``.
``python -m terracemoe_simulator_b200.utils.drift_probe compare A.log B.log`` reports the first
divergent point.  A probe that fails internally disables itself (it must never take a training
run down) unless strict mode is on.

Parity with the reference ``terrace/drift_probe.py`` (:57-91 switches, :171-279 notes, :286-356
contracts, :363-452 offline compare).
"""
from __future__ import annotations

import os
import re
import sys

import torch

PREFIX = "[terrace-drift]"
CMP_RTOL = 1e-6

_CFG = None
_WHERE = {"step": 0, "layer": 0, "call": 0}
_SINK = None            # callable(str) used instead of print (tests)
_DISABLED = False


class DriftProbeMismatch(RuntimeError):
    """A bitwise / reproducibility contract checked by the probe does not hold."""


def reset() -> None:
    global _CFG, _DISABLED
    _CFG = None
    _DISABLED = False
    _WHERE.update(step=0, layer=0, call=0)


def set_sink(fn) -> None:
    global _SINK
    _SINK = fn


def _decide():
    env = os.environ
    on = env.get("TERRACE_DRIFT_PROBE", "").strip().lower() in ("1", "on", "true", "yes")
    ranks = env.get("TERRACE_DRIFT_PROBE_RANKS", "").strip()
    return {
        "on": on,
        "every": max(1, int(env.get("TERRACE_DRIFT_PROBE_EVERY", "1") or 1)),
        "maxcall": int(env.get("TERRACE_DRIFT_PROBE_MAXCALL", "0") or 0),
        "ranks": {int(r) for r in ranks.split(",") if r.strip()} if ranks else None,
        "strict": env.get("TERRACE_DRIFT_PROBE_STRICT", "").strip().lower() in ("1", "on", "true"),
        "chunk": max(1, int(env.get("TERRACE_DRIFT_PROBE_CHUNK", str(1 << 16)) or (1 << 16))),
    }


def _cfg():
    global _CFG
    if _CFG is None:
        _CFG = _decide()
    return _CFG


def enabled() -> bool:
    return _cfg()["on"] and not _DISABLED


def _rank() -> int:
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank()
    except Exception:  # noqa: BLE001
        pass
    return 0


def _live() -> bool:
    if not enabled():
        return False
    c = _cfg()
    call = _WHERE["call"]
    if c["maxcall"] and call > c["maxcall"]:
        return False
    if call % c["every"]:
        return False
    return c["ranks"] is None or _rank() in c["ranks"]


def set_where(step=None, layer=None, call=None) -> None:
    for key, val in (("step", step), ("layer", layer), ("call", call)):
        if val is not None:
            _WHERE[key] = int(val)


def tick_dispatch() -> None:
    _WHERE["call"] += 1


def where() -> str:
    return f"step={_WHERE['step']} layer={_WHERE['layer']} call={_WHERE['call']} rank={_rank()}"


def _emit(line: str) -> None:
    if _SINK is not None:
        _SINK(line)
    else:
        print(line, flush=True)


def _die(exc: Exception, what: str) -> None:
    global _DISABLED
    if _cfg()["strict"]:
        raise exc
    _DISABLED = True
    _emit(f"{PREFIX} probe-disabled what={what} err={type(exc).__name__}")


def _fail(point: str, msg: str) -> None:
    _emit(f"{PREFIX} MISMATCH pt={point} {where()} {msg}")
    if _cfg()["strict"]:
        raise DriftProbeMismatch(f"{point}: {msg}")


def digest(x: torch.Tensor, chunk: int | None = None):
    """``(numel, sum|x|, sum x^2, max|x|)`` in float64, accumulated chunk by chunk."""
    chunk = chunk or _cfg()["chunk"]
    flat = x.detach().reshape(-1)
    n = flat.numel()
    if n == 0:
        return 0, 0.0, 0.0, 0.0
    sabs = ssq = 0.0
    amax = 0.0
    for start in range(0, n, chunk):
        part = flat[start:start + chunk].to(torch.float64)
        sabs += float(part.abs().sum())
        ssq += float((part * part).sum())
        amax = max(amax, float(part.abs().max()))
    return n, sabs, ssq, amax


def digest_int(x: torch.Tensor):
    flat = x.detach().reshape(-1).to(torch.int64)
    if flat.numel() == 0:
        return 0, 0, 0, 0
    return flat.numel(), int(flat.sum()), int(flat.min()), int(flat.max())


def _line(point: str, dt, fields: str) -> str:
    return f"{PREFIX} pt={point} {where()} dt={str(dt).replace('torch.', '')} {fields}"


def note(point: str, x, **_ignored) -> None:
    if not _live():
        return
    try:
        n, sabs, ssq, amax = digest(x)
        _emit(_line(point, x.dtype, f"n={n} sabs={sabs:.17g} ssq={ssq:.17g} amax={amax:.17g}"))
    except Exception as exc:  # noqa: BLE001
        _die(exc, f"note:{point}")


def note_int(point: str, x, **_ignored) -> None:
    if not _live():
        return
    try:
        n, s, lo, hi = digest_int(x)
        _emit(_line(point, x.dtype, f"n={n} isum={s} imin={lo} imax={hi}"))
    except Exception as exc:  # noqa: BLE001
        _die(exc, f"note_int:{point}")


def note_layout(point: str, x, **_ignored) -> None:
    """Layout facts that explain a divergence: shape, strides, contiguity, storage offset."""
    if not _live():
        return
    try:
        _emit(_line(point, x.dtype, f"shape={tuple(x.shape)} stride={tuple(x.stride())} "
                                    f"contig={int(x.is_contiguous())} off={x.storage_offset()}"))
    except Exception as exc:  # noqa: BLE001
        _die(exc, f"note_layout:{point}")


def check_equal(point: str, a, b, note_a: str = "") -> bool:
    """Bitwise contract between two constructions of the same tensor."""
    if not _live():
        return True
    try:
        same = a.shape == b.shape and a.dtype == b.dtype and bool(torch.equal(a, b))
    except Exception as exc:  # noqa: BLE001
        _die(exc, f"check_equal:{point}")
        return True
    if not same:
        diff = "shape/dtype" if (a.shape != b.shape or a.dtype != b.dtype) else \
            f"n_diff={int((a != b).sum())}"
        _fail(point, f"bitwise contract broken {diff} {note_a}".strip())
    return same


def check_reduction(point: str, out, src, index, n_out: int, per=None) -> bool:
    """Is ``out = zeros.index_add(0, index, src)`` reproducible, and how far is it from a
    deterministic fp32 reference (sorted accumulation order)?"""
    if not _live():
        return True
    try:
        again = torch.zeros_like(out).index_add_(0, index, src.to(out.dtype))
        repro = bool(torch.equal(again, out))
        order = torch.argsort(index, stable=True)
        ref = torch.zeros(n_out, *src.shape[1:], dtype=torch.float32, device=src.device)
        ref.index_add_(0, index[order], src[order].float())
        dev = float((out.float() - ref).abs().max()) if out.numel() else 0.0
        _emit(_line(point, out.dtype, f"repro={int(repro)} maxdev={dev:.9g}"))
        if not repro:
            _fail(point, "index_add is not reproducible on this device")
        return repro
    except Exception as exc:  # noqa: BLE001
        _die(exc, f"check_reduction:{point}")
        return True


# ---------------------------------------------------------------------------------------------
# offline comparison of two logs
# ---------------------------------------------------------------------------------------------
_KV = re.compile(r"(\w+)=(\S+)")


def parse_line(line: str):
    if not line.startswith(PREFIX) or " pt=" not in line:
        return None
    return dict(_KV.findall(line[len(PREFIX):]))


def parse_log(path):
    out = []
    with open(path, encoding="utf-8", errors="replace") as f:
        for line in f:
            rec = parse_line(line.strip())
            if rec is not None:
                out.append(rec)
    return out


def _reldiff(a: float, b: float) -> float:
    denom = max(abs(a), abs(b), 1e-300)
    return abs(a - b) / denom


def compare(path_a, path_b, rtol: float = CMP_RTOL, limit: int = 20):
    """Match records by (pt, step, layer, call, rank) and list those whose numeric fields
    differ; the first entry is the first divergence.  Returns the list of mismatch strings."""
    key = lambda r: (r.get("pt"), r.get("step"), r.get("layer"), r.get("call"), r.get("rank"))
    a_recs, b_index = parse_log(path_a), {}
    for r in parse_log(path_b):
        b_index.setdefault(key(r), r)
    problems = []
    for r in a_recs:
        other = b_index.get(key(r))
        if other is None:
            continue
        for field in ("n", "sabs", "ssq", "amax", "isum", "imin", "imax"):
            if field in r and field in other:
                va, vb = float(r[field]), float(other[field])
                exact = field in ("n", "isum", "imin", "imax")
                if (exact and va != vb) or (not exact and _reldiff(va, vb) > rtol):
                    tag = "FIRST-DIVERGENCE" if not problems else "divergence"
                    problems.append(f"{tag} pt={r['pt']} step={r.get('step')} layer={r.get('layer')} "
                                    f"call={r.get('call')} rank={r.get('rank')} {field}: {r[field]} "
                                    f"vs {other[field]}")
                    break
        if len(problems) >= limit:
            break
    return problems


def main(argv) -> int:
    if len(argv) >= 3 and argv[0] == "compare":
        problems = compare(argv[1], argv[2])
        if not problems:
            print("no divergence")
            return 0
        for p in problems:
            print(p)
        return 1
    print("usage: python -m terracemoe_simulator_b200.utils.drift_probe compare A.log B.log")
    return 2


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
