"""Model of the single-MoE-layer step on B200, checked against the measured steps.

On the reference machine the step-level gate fails: communication hides behind other work in
ways no one-parameter overlap model captures (``sim/validate.py``, ``sim/overlap.py``).  On B200
the layer has two schedules whose structure is known, so each gets its own sum:

    serial   (remote-read arms, ``TERRACE_EP_OVERLAP=0``): nothing overlaps,
             step = GEMMs + memory-bound kernels + 2 x (dispatch + combine)

    overlap  (default): the dispatch leaves in chunks on a side stream and the return leg rides in
             the second GEMM's epilogue, so per direction only ``phase.ChunkedSchedule.exposed_ms``
             stays visible: the first chunk's share of the dispatch, whatever a later chunk's
             transfer exceeds the GEMM time it hides under, and the local reduction
             step = GEMMs + memory-bound kernels + exposed(forward) + exposed(backward)

The GEMM term is priced from the kernels' measured throughput (long groups, with the 128-row tile
quantisation of short groups and the weight-gradient kernel's epilogue exposure), scaled by the
SM clock: the kernel figures hold at the clock the kernels reach when timed alone, and a step
under the 1 kW power cap runs slower the busier it keeps the GPU (1515 MHz on one GPU, where
nothing ever waits; 1736 MHz on four; 1897 MHz on eight), so every run carries the median
clock sampled during it.  The GEMM time follows the square root of the clock ratio, not the
ratio itself: the sampler sees the waits, where the clock recovers, as much as the GEMMs (fit:
the GEMMs of the one-GPU launch list, 2.63 ms, and of the 4-GPU phase spans, 2.15 ms).  The
constants that are fitted rather than measured (the two elementwise remainders, the hidden share
of the return transfer, the two-hop relay) come from the 1-, 2- and 4-GPU runs; the 8-GPU run is
a prediction.  The communication term is the calibrated call model
(``calibrate.b200_nvswitch``).  Every measured number is read from a JSON file
(``sim/data/b200_layer_bench.json`` by default; ``--bench FILE`` takes the lines ``bench.py``
printed), none is in this source.

``python -m terracemoe_simulator_b200.sim.b200_step`` prints model against measurement for every
measured (GPUs, path, schedule) and the gate (every configuration within 10 %).

No counterpart in the reference (its phase model refuses to return a number, ``sim/phase.py``).
"""
from __future__ import annotations

import json
import os

from ._text import Column, render_table
from .calibrate import b200_nvswitch
from .core import MoEGeometry, one_hop_call, two_hop_call
from .phase import ChunkedSchedule

GATE = 0.10
DATA = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "b200_layer_bench.json")

# Layer of the headline benchmark: d_model 4096, 64 experts of hidden 1408, top-6, M = 2,
# 4096 tokens per GPU.
HIDDEN, D_EXPERT, N_EXPERTS, TOP_K, TOP_GROUPS, TOKENS = 4096, 1408, 64, 6, 2, 4096
TILE_ROWS, SEG_ALIGN = 128, 64
SCHEDULES = ("serial", "overlap")


# ---- measurements ---------------------------------------------------------------------------------
def _runs_from_bench_lines(lines) -> list:
    """``bench.py`` JSON lines -> run records ``{n_gpus, rpn, chunks, paths: {name: ms}}``; the
    ``*_pull`` paths of a line are the serial arms of the same run."""
    runs = []
    for d in lines:
        if d.get("impl", "ours") != "ours" or "paths" not in d:
            continue
        runs.append({"n_gpus": d["n_gpus"], "rpn": d["config"].get("rpn", 1),
                     "chunks": d.get("impl_detail", {}).get("chunks", 2),
                     "schedule": d.get("impl_detail", {}).get("schedule", "overlap"),
                     "paths": {name: p["ms_per_step"] for name, p in d["paths"].items()}})
    return runs


def load_bench(path: str | None = None) -> dict:
    """The measured steps and kernel figures: either the committed file (``runs`` + ``kernels``)
    or a file of ``bench.py`` output lines (kernel figures then come from the committed file)."""
    with open(DATA) as f:
        shipped = json.load(f)
    if path is None or os.path.abspath(path) == DATA:
        return shipped
    with open(path) as f:
        text = f.read().strip()
    try:
        given = json.loads(text)
    except ValueError:                                   # one JSON object per line
        given = [json.loads(row) for row in text.splitlines() if row.startswith("{")]
    if isinstance(given, dict) and "runs" in given:
        return {**shipped, **given}
    lines = given if isinstance(given, list) else [given]
    return {**shipped, "runs": _runs_from_bench_lines(lines), "source": path}


def measured_steps(bench: dict | None = None) -> dict:
    """``{(GPUs, ranks per group, path, schedule): ms per step}``."""
    bench = bench or load_bench()
    out = {}
    for run in bench["runs"]:
        default = run.get("schedule", "overlap")
        for name, ms in run["paths"].items():
            serial = name.endswith("_pull")
            path = name[:-5] if serial else name
            schedule = "serial" if serial or default == "serial" else "overlap"
            if path == "local":
                schedule = "serial"
            out[run["n_gpus"], run["rpn"], path, schedule] = ms
    return out


class _Kernels:
    """Kernel-level figures of the data file, by attribute."""

    def __init__(self, table: dict):
        self.__dict__.update(table)


def kernels(bench: dict | None = None) -> _Kernels:
    return _Kernels((bench or load_bench())["kernels"])


# ---- terms ------------------------------------------------------------------------------------------
def tile_efficiency(rows_per_expert: float) -> float:
    """Share of the MMA rows that carry data when a group of ``rows_per_expert`` rows (random
    around that mean, padded to 64) is cut into 128-row tiles: half a tile is wasted on average
    once per group."""
    padded = rows_per_expert + SEG_ALIGN / 2.0
    slots = padded + TILE_ROWS / 2.0 - SEG_ALIGN / 2.0
    return min(1.0, rows_per_expert / slots)


def gemm_ms(n_gpus: int, kern: _Kernels | None = None, sm_mhz: float | None = None) -> dict:
    """Forward and backward grouped GEMM time of one step on each GPU, at SM clock ``sm_mhz``
    (default: the clock of the kernels timed alone)."""
    kern = kern or kernels()
    rows = TOKENS * TOP_K                              # rows per GPU after dispatch (balanced)
    per_expert = rows / (N_EXPERTS // n_gpus)
    flops_fwd = 2.0 * rows * HIDDEN * D_EXPERT * 3     # gate, up, down
    eff = tile_efficiency(per_expert)
    fwd_dgrad_tflops = kern.tflops_fwd_dgrad_long * eff
    # weight gradient: its epilogue shows with short groups, 1/T = 1/T_long + c / rows
    c = (1.0 / kern.tflops_wgrad_short - 1.0 / kern.tflops_wgrad_long) * kern.wgrad_short_rows
    wgrad_tflops = 1.0 / (1.0 / kern.tflops_wgrad_long + c / per_expert)
    derate = (kern.gemm_alone_sm_mhz / sm_mhz) ** kern.clock_exponent if sm_mhz else 1.0
    fwd = derate * flops_fwd / (fwd_dgrad_tflops * 1e9)
    bwd = derate * (flops_fwd / (fwd_dgrad_tflops * 1e9) + flops_fwd / (wgrad_tflops * 1e9))
    return {"rows_per_expert": per_expert, "tile_efficiency": eff,
            "fwd_dgrad_tflops": fwd_dgrad_tflops, "wgrad_tflops": wgrad_tflops,
            "fwd_ms": fwd, "bwd_ms": bwd, "ms": fwd + bwd}


def comm_ms(n_gpus: int, rpn: int, path: str, kern: _Kernels | None = None) -> float:
    """Dispatch + combine of one direction pair (there and back), ms."""
    kern = kern or kernels()
    if n_gpus == 1:
        return kern.local_dispatch_combine_ms
    n_groups = max(n_gpus // rpn, 2)
    geom = MoEGeometry(f"b200x{n_gpus}", n_groups, max(n_gpus // n_groups, 1), TOP_K, TOP_GROUPS,
                       H=HIDDEN, seq=TOKENS, gbs=n_gpus * TOKENS)
    call = one_hop_call if path == "one_hop" else two_hop_call
    return 2.0 * call(b200_nvswitch(R=geom.R), geom)


def local_reduce_ms(kern: _Kernels | None = None) -> float:
    """Gate-weighted reduction of k rows per token from this GPU's own return slots."""
    kern = kern or kernels()
    moved = (TOP_K + 1) * TOKENS * HIDDEN * 2.0
    return moved / (kern.hbm_copy_gbps * 1e6)


def run_clock(n_gpus: int, bench: dict | None = None):
    """Median SM clock sampled during the measured run on ``n_gpus`` GPUs (None if not recorded)."""
    for run in (bench or load_bench())["runs"]:
        if run["n_gpus"] == n_gpus and run.get("sm_mhz"):
            return float(run["sm_mhz"])
    return None


def predict_ms(n_gpus: int, rpn: int, path: str, schedule: str = "overlap", chunks: int = 2,
               bench: dict | None = None, sm_mhz: float | None = None) -> dict:
    """``sm_mhz``: SM clock of the step (default: the one sampled during the measured run at
    this GPU count, else the clock of the kernels timed alone)."""
    if schedule not in SCHEDULES:
        raise ValueError(f"schedule must be one of {SCHEDULES}")
    kern = kernels(bench)
    g = gemm_ms(n_gpus, kern, sm_mhz or run_clock(n_gpus, bench))
    pair = comm_ms(n_gpus, rpn, path, kern)
    if n_gpus == 1:
        exposed = 2.0 * pair
        total = g["ms"] + kern.elementwise_local_ms + exposed
    elif schedule == "serial":
        exposed = 2.0 * pair                                    # forward and backward
        total = g["ms"] + kern.elementwise_fused_ms + exposed
    else:
        plan = ChunkedSchedule(chunks=chunks, local_reduce_ms=local_reduce_ms(kern),
                               return_hidden=kern.return_hidden)
        one_way = 0.5 * pair
        extra = kern.two_hop_relay_ms if path == "two_hop" else 0.0
        exposed = (plan.exposed_ms(one_way, g["fwd_ms"], one_way)
                   + plan.exposed_ms(one_way, g["bwd_ms"], one_way) + 2.0 * extra)
        total = g["ms"] + kern.elementwise_fused_ms + exposed
    return {"gemm_ms": g["ms"], "comm_ms": pair, "exposed_ms": exposed, "total_ms": total,
            "gemm": g}


# ---- gate -------------------------------------------------------------------------------------------
def validate(verbose: bool = True, bench: dict | None = None):
    bench = bench or load_bench()
    rows = []
    for (n, rpn, path, schedule), measured in sorted(measured_steps(bench).items()):
        p = predict_ms(n, rpn, path, schedule, bench=bench)
        rows.append((n, rpn, path, schedule, measured, p["total_ms"], p["gemm_ms"],
                     p["exposed_ms"], p["total_ms"] / measured - 1.0))
    worst = max((abs(r[-1]) for r in rows), default=0.0)
    fitted = set(bench["kernels"].get("fitted_on_gpus", []))
    predicted = [abs(r[-1]) for r in rows if r[0] not in fitted]
    ok = bool(rows) and worst <= GATE
    if verbose:
        cols = [Column("GPUs", "%4d", lambda r: r[0]), Column("rpn", "%4d", lambda r: r[1]),
                Column("path", "%-8s", lambda r: r[2]), Column("schedule", "%-8s", lambda r: r[3]),
                Column("measured", "%9.2f", lambda r: r[4]), Column("model", "%9.2f", lambda r: r[5]),
                Column("GEMMs", "%9.2f", lambda r: r[6]), Column("exposed", "%9.2f", lambda r: r[7]),
                Column("err", "%7s", lambda r: "%+.1f%%" % (100 * r[8])),
                Column("", "%-9s", lambda r: "fitted" if r[0] in fitted else "predicted")]
        print("single-MoE-layer step on B200: model against measurement (ms per step)")
        print("\n".join(render_table(cols, rows)))
        print("worst error %.1f%% (gate %.0f%%); worst of the %d predicted rows %.1f%%"
              % (100 * worst, 100 * GATE, len(predicted), 100 * max(predicted, default=0.0)))
        print("**B200 step gate %s**" % ("PASS" if ok else "FAIL"))
    return ok, {"worst": worst, "rows": rows, "worst_predicted": max(predicted, default=0.0)}


def overlap_gain(verbose: bool = True, bench: dict | None = None) -> list:
    """What the overlap schedule removes, measured and modelled: serial - overlap per
    (GPUs, path)."""
    bench = bench or load_bench()
    steps = measured_steps(bench)
    rows = []
    for (n, rpn, path, schedule), ms in sorted(steps.items()):
        if schedule != "overlap" or (n, rpn, path, "serial") not in steps:
            continue
        model = (predict_ms(n, rpn, path, "serial", bench=bench)["total_ms"]
                 - predict_ms(n, rpn, path, "overlap", bench=bench)["total_ms"])
        rows.append((n, rpn, path, steps[n, rpn, path, "serial"] - ms, model))
    if verbose:
        print("time removed by the overlap schedule (serial - overlap, ms per step)")
        cols = [Column("GPUs", "%4d", lambda r: r[0]), Column("rpn", "%4d", lambda r: r[1]),
                Column("path", "%-8s", lambda r: r[2]), Column("measured", "%9.2f", lambda r: r[3]),
                Column("model", "%9.2f", lambda r: r[4])]
        print("\n".join(render_table(cols, rows)))
    return rows


def path_ratios(verbose: bool = True, bench: dict | None = None) -> list:
    """two-hop / one-hop step time per (GPUs, schedule), measured and modelled: the step-level
    counterpart of the call-level ratio gate (``sim/validate_b200.py``)."""
    bench = bench or load_bench()
    steps = measured_steps(bench)
    fitted = set(bench["kernels"].get("fitted_on_gpus", []))
    rows = []
    for (n, rpn, path, schedule), one in sorted(steps.items()):
        two = steps.get((n, rpn, "two_hop", schedule))
        if path != "one_hop" or two is None:
            continue
        model = (predict_ms(n, rpn, "two_hop", schedule, bench=bench)["total_ms"]
                 / predict_ms(n, rpn, "one_hop", schedule, bench=bench)["total_ms"])
        rows.append((n, rpn, schedule, two / one, model, model / (two / one) - 1.0, n in fitted))
    if verbose:
        print("two-hop / one-hop step time")
        cols = [Column("GPUs", "%4d", lambda r: r[0]), Column("rpn", "%4d", lambda r: r[1]),
                Column("schedule", "%-8s", lambda r: r[2]), Column("measured", "%9.3f", lambda r: r[3]),
                Column("model", "%9.3f", lambda r: r[4]),
                Column("err", "%7s", lambda r: "%+.1f%%" % (100 * r[5])),
                Column("", "%-9s", lambda r: "fitted" if r[6] else "predicted")]
        print("\n".join(render_table(cols, rows)))
    return rows


def main(argv=None) -> None:
    import argparse
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--bench", default=None,
                    help="file of bench.py output lines (default: the committed measurements)")
    ns = ap.parse_args(argv)
    bench = load_bench(ns.bench)
    validate(bench=bench)
    print()
    overlap_gain(bench=bench)
    print()
    path_ratios(bench=bench)


if __name__ == "__main__":
    main()
