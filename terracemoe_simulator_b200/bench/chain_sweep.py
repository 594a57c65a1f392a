"""Single-device cost of the arrival step over pair count and hidden width.

Times ``k1_arrival`` (the sm_100a kernel when the native library is loaded) and its PyTorch
specification ``k1_arrival_ref`` over pairs in {1024 .. 65536} and H in {1024 .. 8192} with
quota 6, 4 experts per rank and a group of 64 ranks, the shapes of the reference's sweep
(``bench/chain_sweep.py:50-118``), and fits ``ms = fixed + pairs * per_pair`` per width.
``sim.machine`` holds the reference machine's result (28.6 ns of index work per pair and a
1469 GB/s row gather); this script produces the same two constants for the device it runs on.

    python -m terracemoe_simulator_b200.bench.chain_sweep --out chain.json
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time

import torch

PAIRS = [1024, 2048, 4096, 8192, 16384, 32768, 65536]
WIDTHS = [1024, 2048, 4096, 8192]


def time_ms(fn, n: int, device: torch.device) -> float:
    if device.type == "cuda":
        out = []
        for _ in range(n):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            out.append(a.elapsed_time(b))
        return statistics.median(out)
    out = []
    for _ in range(n):
        t0 = time.perf_counter()
        fn()
        out.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(out)


def line_fit(xs, ys):
    """Least-squares ``y = a + b x``; returns (a, b)."""
    n = len(xs)
    mx, my = sum(xs) / n, sum(ys) / n
    sxx = sum((x - mx) ** 2 for x in xs)
    b = sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / max(sxx, 1e-30)
    return my - b * mx, b


def sweep(device, pairs_list, widths, quota, epr, rpn, calls, use_ref_only=False):
    from .. import ops
    from ..ops.refs import k1_arrival_ref
    rows = []
    for H in widths:
        for pairs in pairs_list:
            n_rows = max(1, pairs // quota)
            rx = torch.randn(n_rows, H, device=device).to(torch.bfloat16)
            rslot = torch.randint(0, rpn * epr, (n_rows, quota), device=device).sort(dim=1).values
            rgate = torch.randn(n_rows, quota, device=device).to(torch.bfloat16)
            ref = lambda: k1_arrival_ref(rx, rslot, rgate, quota, epr, rpn)       # noqa: E731
            live = lambda: ops.k1_arrival(rx, rslot, rgate, quota=quota, epr=epr, rpn=rpn)  # noqa: E731
            for fn in (ref, live):
                fn()
            row = {"H": H, "pairs": n_rows * quota, "ref_ms": time_ms(ref, calls, device)}
            if not use_ref_only:
                row["live_ms"] = time_ms(live, calls, device)
                row["live_over_ref"] = row["live_ms"] / max(row["ref_ms"], 1e-12)
            rows.append(row)
    return rows


def fits(rows, key):
    out = {}
    for H in sorted({r["H"] for r in rows}):
        sel = [r for r in rows if r["H"] == H and key in r]
        if len(sel) >= 2:
            fixed, per = line_fit([r["pairs"] for r in sel], [r[key] for r in sel])
            out[H] = {"fixed_ms": fixed, "ns_per_pair": per * 1e6,
                      "gather_gbs": (2 * H * 2) / max(per * 1e-3, 1e-30) / 1e9}
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--out", required=True)
    ap.add_argument("--pairs", type=int, nargs="+", default=PAIRS)
    ap.add_argument("--hidden", type=int, nargs="+", default=WIDTHS)
    ap.add_argument("--quota", type=int, default=6)
    ap.add_argument("--epr", type=int, default=4)
    ap.add_argument("--rpn", type=int, default=64)
    ap.add_argument("--calls", type=int, default=9)
    ap.add_argument("--cpu", action="store_true")
    args = ap.parse_args(argv)
    device = torch.device("cuda" if torch.cuda.is_available() and not args.cpu else "cpu")
    from .. import ops
    rows = sweep(device, args.pairs, args.hidden, args.quota, args.epr, args.rpn, args.calls)
    for r in rows:
        print("H=%5d pairs=%6d  ref %8.4f ms  live %8.4f ms  live/ref %.3f"
              % (r["H"], r["pairs"], r["ref_ms"], r["live_ms"], r["live_over_ref"]), flush=True)
    payload = {"device": str(device), "native": bool(ops.custom_ops_enabled()), "rows": rows,
               "fit_ref": fits(rows, "ref_ms"), "fit_live": fits(rows, "live_ms")}
    with open(args.out, "w", encoding="utf-8") as fh:
        json.dump(payload, fh, indent=1)
    print(f"wrote {args.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
