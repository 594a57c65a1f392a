"""Additive model of the single-MoE-layer step on B200, checked against the measured steps.

On the reference machine the step-level gate fails: communication hides behind other work in
ways no one-parameter overlap model captures (``sim/validate.py``, ``sim/overlap.py``).  On B200
the fused layer has, today, no overlap at all between its phases, so the plain sum should hold:

    step = grouped GEMMs (forward + backward, priced from the measured kernel throughput with
           the 128-row tile quantisation of short groups)
         + memory-bound kernels around them (measured, independent of the GPU count because the
           tokens per GPU are fixed)
         + 2 x (dispatch + combine)            forward and backward, from the calibrated
                                               ``calibrate.b200_nvswitch`` call model

``python -m terracemoe_simulator_b200.sim.b200_step`` prints model against measurement for the
1-, 2- and 8-GPU runs of ``bench.py`` and the gate (every configuration within 10 %).  A gate
that starts failing after dispatch / combine get overlapped with the GEMMs is the expected
outcome of that optimisation, and the place to add the overlap term.

No counterpart in the reference (its phase model refuses to return a number, ``sim/phase.py``).
"""
from __future__ import annotations

from .calibrate import b200_nvswitch
from .core import MoEGeometry, one_hop_call, two_hop_call

GATE = 0.10

# Layer of the headline benchmark: d_model 4096, 64 experts of hidden 1408, top-6, M = 2,
# 4096 tokens per GPU.
HIDDEN, D_EXPERT, N_EXPERTS, TOP_K, TOP_GROUPS, TOKENS = 4096, 1408, 64, 6, 2, 4096

# Measured kernel throughput with long groups (8 local experts x 3072 rows; CUDA events,
# ``bench/kernel_cases.py``), TFLOPS: forward / dgrad kernels and the weight-gradient kernel.
TFLOPS_FWD_DGRAD_LONG = 1300.0
TFLOPS_WGRAD_LONG = 1240.0
# The weight-gradient kernel reduces over a group's rows: with short groups its main loop is
# short and the epilogue shows.  Measured 939 TFLOPS at 384 rows per expert.
WGRAD_SHORT_ROWS, TFLOPS_WGRAD_SHORT = 384.0, 939.0
TILE_ROWS, SEG_ALIGN = 128, 64
# Memory-bound kernels of one step (router, plan, scatter, combine and their backward parts):
# measured 0.45 ms on one GPU; the fused path replaces scatter / combine by push / pull kernels
# that are priced inside the dispatch + combine term, which leaves the GEMM-side remainder
# (SwiGLU backward 0.08, router and plan 0.06, padding and small elementwise kernels 0.1).
ELEMENTWISE_LOCAL_MS = 0.45
ELEMENTWISE_FUSED_MS = 0.25

# (GPUs, ranks per group, path) -> measured ms per step (bench.py, CUDA events, max over ranks)
MEASURED_MS = {
    (1, 1, "local"): 3.27,
    (2, 1, "one_hop"): 3.46,
    (2, 1, "two_hop"): 3.31,
    (8, 2, "one_hop"): 3.77,
    (8, 2, "two_hop"): 3.70,
}
# dispatch + combine measured alone on one GPU (local scatter + combine), ms
LOCAL_DISPATCH_COMBINE_MS = 0.13


def tile_efficiency(rows_per_expert: float) -> float:
    """Share of the MMA rows that carry data when a group of ``rows_per_expert`` rows (random
    around that mean, padded to 64) is cut into 128-row tiles: half a tile is wasted on average
    once per group."""
    padded = rows_per_expert + SEG_ALIGN / 2.0
    slots = padded + TILE_ROWS / 2.0 - SEG_ALIGN / 2.0
    return min(1.0, rows_per_expert / slots)


def gemm_ms(n_gpus: int) -> dict:
    """Forward + backward grouped GEMM time of one step on each GPU."""
    rows = TOKENS * TOP_K                              # rows per GPU after dispatch (balanced)
    local_experts = N_EXPERTS // n_gpus
    per_expert = rows / local_experts
    flops_fwd = 2.0 * rows * HIDDEN * D_EXPERT * 3     # gate, up, down
    eff = tile_efficiency(per_expert)
    fwd_dgrad_tflops = TFLOPS_FWD_DGRAD_LONG * eff
    # weight gradient: interpolate its epilogue exposure as 1/T = 1/T_long + c / rows
    c = (1.0 / TFLOPS_WGRAD_SHORT - 1.0 / TFLOPS_WGRAD_LONG) * WGRAD_SHORT_ROWS
    wgrad_tflops = 1.0 / (1.0 / TFLOPS_WGRAD_LONG + c / per_expert)
    t_fwd_dgrad = 2.0 * flops_fwd / (fwd_dgrad_tflops * 1e12) * 1e3
    t_wgrad = flops_fwd / (wgrad_tflops * 1e12) * 1e3
    return {"rows_per_expert": per_expert, "tile_efficiency": eff,
            "fwd_dgrad_tflops": fwd_dgrad_tflops, "wgrad_tflops": wgrad_tflops,
            "ms": t_fwd_dgrad + t_wgrad}


def comm_ms(n_gpus: int, rpn: int, path: str) -> float:
    """Dispatch + combine of one direction pair (there and back), ms."""
    if n_gpus == 1:
        return LOCAL_DISPATCH_COMBINE_MS
    n_groups = max(n_gpus // rpn, 2)
    geom = MoEGeometry(f"b200x{n_gpus}", n_groups, max(n_gpus // n_groups, 1), TOP_K, TOP_GROUPS,
                       H=HIDDEN, seq=TOKENS, gbs=n_gpus * TOKENS)
    cluster = b200_nvswitch(R=geom.R)
    call = one_hop_call if path == "one_hop" else two_hop_call
    return 2.0 * call(cluster, geom)                   # dispatch + combine


# measured copy bandwidth of one B200 (STREAM-style), GB/s: prices the local reduction that
# replaces the remote pull when the expert GEMM's epilogue delivers the rows
HBM_COPY_GBPS = 6556.0


def local_reduce_ms() -> float:
    """Gate-weighted reduction of k rows per token from this GPU's own return slots."""
    read = TOKENS * TOP_K * HIDDEN * 2.0
    write = TOKENS * HIDDEN * 2.0
    return (read + write) / (HBM_COPY_GBPS * 1e6)


def predict_ms(n_gpus: int, rpn: int, path: str, epilogue_push: bool = False) -> dict:
    """``epilogue_push`` (one-hop only): the combine transfer rides in the second GEMM's epilogue
    and is assumed hidden under it; what stays exposed of each dispatch + combine pair is the
    dispatch and a local reduction.  A forecast written down before the first run of that path."""
    g = gemm_ms(n_gpus)
    c = comm_ms(n_gpus, rpn, path)
    if n_gpus == 1:
        total = g["ms"] + ELEMENTWISE_LOCAL_MS + LOCAL_DISPATCH_COMBINE_MS
    elif epilogue_push:
        if path != "one_hop":
            raise ValueError("the scattering epilogue exists for the one-hop path only")
        c = 0.5 * c + local_reduce_ms()
        total = g["ms"] + ELEMENTWISE_FUSED_MS + 2.0 * c
    else:
        total = g["ms"] + ELEMENTWISE_FUSED_MS + 2.0 * c      # forward and backward
    return {"gemm_ms": g["ms"], "comm_ms": c, "total_ms": total, "gemm": g}


PIPELINE_GEMM_TAIL = 0.03      # extra tail of the shorter per-slice GEMM launches (n = 2, 8 GPUs)


def predict_pipelined_ms(n_gpus: int, rpn: int, path: str, slices: int = 2) -> dict:
    """Token-sliced pipeline: while one slice computes, another dispatches or combines, so as long
    as a slice's GEMMs outlast its communication only the first dispatch and the last combine
    stay exposed, 1 / slices of the total; the GEMMs pay a small tail for their shorter launches.
    A forecast written down before the first run of that path."""
    if n_gpus == 1 or slices < 2:
        return predict_ms(n_gpus, rpn, path)
    g = gemm_ms(n_gpus)
    c = comm_ms(n_gpus, rpn, path)
    gemm = g["ms"] * (1.0 + PIPELINE_GEMM_TAIL)
    per_slice_comm, per_slice_gemm = 2.0 * c / slices, gemm / slices
    hidden_ok = per_slice_gemm >= per_slice_comm
    exposed = 2.0 * c / slices if hidden_ok else 2.0 * c - (slices - 1) * per_slice_gemm
    return {"gemm_ms": gemm, "comm_ms": c, "total_ms": gemm + ELEMENTWISE_FUSED_MS + exposed,
            "hidden": hidden_ok}


def forecast_epilogue_push(verbose: bool = True) -> list:
    """Expected one-hop step with the combine folded into the GEMM, next to today's model and
    measurement.  The additive model reads 2-8 % low, so the forecast is scaled by the measured /
    modelled ratio of the same configuration."""
    rows = []
    for (n, rpn, path), measured in sorted(MEASURED_MS.items()):
        if path != "one_hop":
            continue
        now = predict_ms(n, rpn, path)["total_ms"]
        then = predict_ms(n, rpn, path, epilogue_push=True)["total_ms"]
        rows.append((n, rpn, measured, now, then, then * measured / now))
    if verbose:
        print("one-hop step with the combine transfer in the GEMM epilogue: forecast")
        print("%4s %4s %9s %9s %9s %12s" % ("GPUs", "rpn", "measured", "model", "forecast",
                                            "scaled (ms)"))
        for n, rpn, m, now, then, scaled in rows:
            print("%4d %4d %9.2f %9.2f %9.2f %12.2f" % (n, rpn, m, now, then, scaled))
    return rows


def validate(verbose: bool = True):
    rows, worst = [], 0.0
    for (n, rpn, path), measured in sorted(MEASURED_MS.items()):
        p = predict_ms(n, rpn, path)
        err = (p["total_ms"] - measured) / measured
        worst = max(worst, abs(err))
        rows.append((n, rpn, path, measured, p["total_ms"], p["gemm_ms"], p["comm_ms"], err))
    ok = worst <= GATE
    if verbose:
        print("single-MoE-layer step on B200: additive model against measurement")
        print("%4s %4s %-8s %9s %9s %9s %9s %7s" % ("GPUs", "rpn", "path", "measured", "model",
                                                    "GEMMs", "d+c", "err"))
        for n, rpn, path, m, t, g, c, e in rows:
            print("%4d %4d %-8s %9.2f %9.2f %9.2f %9.2f %+6.1f%%" % (n, rpn, path, m, t, g, c,
                                                                     100 * e))
        print("worst error %.1f%% (gate %.0f%%)" % (100 * worst, 100 * GATE))
        print("**B200 step gate %s**" % ("PASS" if ok else "FAIL"))
    return ok, {"worst": worst, "rows": rows}


def forecast_pipeline(verbose: bool = True, slices: int = 2) -> list:
    rows = []
    for (n, rpn, path), measured in sorted(MEASURED_MS.items()):
        if n == 1:
            continue
        now = predict_ms(n, rpn, path)["total_ms"]
        then = predict_pipelined_ms(n, rpn, path, slices)["total_ms"]
        rows.append((n, rpn, path, measured, now, then, then * measured / now))
    if verbose:
        print("step with %d token slices on %d streams: forecast" % (slices, slices))
        print("%4s %4s %-8s %9s %9s %9s %12s" % ("GPUs", "rpn", "path", "measured", "model",
                                                 "forecast", "scaled (ms)"))
        for n, rpn, path, m, now, then, scaled in rows:
            print("%4d %4d %-8s %9.2f %9.2f %9.2f %12.2f" % (n, rpn, path, m, now, then, scaled))
    return rows


def main() -> None:
    validate()
    print()
    forecast_epilogue_push()
    print()
    forecast_pipeline()


if __name__ == "__main__":
    main()
