"""Expert-FFN compute pricing from measured GEMM throughput.

Two tables: the reference's Ascend 910C square-GEMM roofline with eight non-square expert
shapes (which settle the index rule: geometric mean of the three dimensions, 6.4 % median
error), and the B200 numbers of this repository's tcgen05 grouped GEMM.  ``expert_ffn`` prices
one layer's routed experts on one rank; compute is never added to communication here because
their overlap is unresolved.

Parity with the reference ``sim/compute.py`` (tables :65-84, ``achieved_tflops`` / ``index_dims``
/ ``efficiency_bracket`` :103-139, ``expert_ffn`` :142-178, ``comm_share_upper_bound`` :181-190).
"""
from __future__ import annotations

import bisect

GEMM_TFLOPS = [(1024, 141.6), (2048, 271.1), (4096, 327.4), (8192, 296.7), (12288, 291.4),
               (16384, 319.2)]
PEAK_TFLOPS = max(t for _, t in GEMM_TFLOPS)
INDEX_RULES = ("min_dim", "geometric_mean", "rows")
NONSQUARE_TFLOPS = {
    (1536, 2048, 5504): 309.7, (1536, 4096, 11008): 326.7, (1536, 7168, 2048): 328.3,
    (3072, 2048, 5504): 324.8, (3072, 4096, 11008): 335.9, (3072, 7168, 2048): 338.0,
    (6144, 2048, 5504): 331.4, (6144, 4096, 11008): 330.7,
}
INDEX_RULE = "geometric_mean"
INDEX_RULE_ERROR = {"median_abs": 0.064, "bias": -0.064, "worst": 0.109}

# B200, this repository's grouped GEMM (24576 rows, d_model 4096, expert width 1408), TFLOPS by
# number of local experts; cuBLAS 8192^3 on the same GPU for scale.
B200_GROUPED_TFLOPS = {
    8: {"fwd_swiglu": 1258.9, "fwd": 1306.8, "gemm2": 1186.8, "dgrad": 1301.4, "wgrad": 1259.6},
    64: {"fwd_swiglu": 1034.2, "fwd": 1071.1, "gemm2": 992.0, "dgrad": 1026.3, "wgrad": 738.1},
}
B200_CUBLAS_8192_TFLOPS = 1604.8


def achieved_tflops(dim: float, table=None) -> float:
    pts = table or GEMM_TFLOPS
    xs = [x for x, _ in pts]
    if dim <= xs[0]:
        return pts[0][1]
    if dim >= xs[-1]:
        return pts[-1][1]
    i = bisect.bisect_right(xs, dim)
    (x0, y0), (x1, y1) = pts[i - 1], pts[i]
    return y0 + (y1 - y0) * (dim - x0) / (x1 - x0)


def index_dims(rows: int, hidden: int, d_expert: int) -> dict:
    return {"min_dim": float(min(rows, hidden, d_expert)),
            "geometric_mean": (rows * hidden * d_expert) ** (1.0 / 3.0), "rows": float(rows)}


def efficiency_bracket(rows: int, hidden: int, d_expert: int) -> dict:
    per_rule = {k: achieved_tflops(v) for k, v in index_dims(rows, hidden, d_expert).items()}
    lo, hi = min(per_rule.values()), max(per_rule.values())
    return {"per_rule": per_rule, "lo": lo, "hi": hi, "spread": hi / lo}


def expert_ffn(tokens_per_rank: int, k: int, n_experts: int, ep: int, hidden: int,
               d_expert: int, n_mats: int = 2, backward: bool = False) -> dict:
    """Exact FLOPs of the routed experts of one rank and their time on platform A."""
    experts_local = max(n_experts // ep, 1)
    rows = max(tokens_per_rank * k // experts_local, 1)
    flops = 2.0 * rows * hidden * d_expert * n_mats * experts_local * (2.0 if backward else 1.0)
    br = efficiency_bracket(rows, hidden, d_expert)
    tflops = br["per_rule"][INDEX_RULE]
    ms = flops / (tflops * 1e12) * 1e3
    worst = INDEX_RULE_ERROR["worst"]
    return {"flops": flops, "rows_per_expert": rows, "experts_local": experts_local,
            "tflops": tflops, "ms": ms, "ms_lo": ms * (1.0 - worst), "ms_hi": ms * (1.0 + worst),
            "rule": INDEX_RULE, "rule_error": dict(INDEX_RULE_ERROR),
            "ms_fast": flops / (br["hi"] * 1e12) * 1e3, "ms_slow": flops / (br["lo"] * 1e12) * 1e3,
            "tflops_bracket": (br["lo"], br["hi"]), "assumption_spread": br["spread"],
            "efficiency_vs_peak": tflops / PEAK_TFLOPS}


def expert_ffn_b200(tokens_per_rank: int, k: int, n_experts: int, ep: int, hidden: int,
                    d_expert: int, backward: bool = False) -> dict:
    """Same ledger priced with the B200 grouped-GEMM measurements (three matrices: gate, up,
    down); throughput interpolated in the number of local experts."""
    experts_local = max(n_experts // ep, 1)
    rows = tokens_per_rank * k
    flops = 2.0 * rows * hidden * d_expert * 3 * (3.0 if backward else 1.0)
    pts = sorted((e, (v["fwd_swiglu"] * 2 + v["gemm2"]) / 3.0 if not backward else
                  (v["fwd_swiglu"] * 2 + v["gemm2"] + v["dgrad"] * 3 + v["wgrad"] * 3) / 9.0)
                 for e, v in B200_GROUPED_TFLOPS.items())
    tflops = achieved_tflops(float(experts_local), pts)
    return {"flops": flops, "experts_local": experts_local, "tflops": tflops,
            "ms": flops / (tflops * 1e12) * 1e3}


def comm_share_upper_bound(comm_ms: float, compute_ms: float) -> float:
    total = comm_ms + compute_ms
    return comm_ms / total if total > 0 else float("nan")


def main() -> None:
    print("Measured bf16 GEMM roofline, platform A (256 samples per size):")
    for n, t in GEMM_TFLOPS:
        print("  %6d  %6.1f TFLOPS  %3.0f%% of peak" % (n, t, 100 * t / PEAK_TFLOPS))
    print("\nMeasured expert-FFN shapes, and what each index rule would have said:")
    print("  %-22s %9s %8s %8s %8s" % ("rows x hidden x d_exp", "measured", "geo-mean", "min-dim",
                                       "rows"))
    for shape, meas in sorted(NONSQUARE_TFLOPS.items()):
        per = efficiency_bracket(*shape)["per_rule"]
        print("  %-22s %9.1f %8.0f %8.0f %8.0f" % ("%d x %d x %d" % shape, meas,
                                                   per["geometric_mean"], per["min_dim"],
                                                   per["rows"]))
    print("  geometric mean is the rule in use: %.1f%% median error, worst %.1f%%"
          % (100 * INDEX_RULE_ERROR["median_abs"], 100 * INDEX_RULE_ERROR["worst"]))
    print("\nExpert-FFN forward, one layer, one rank: T=4096, k=6, E=128, EP=128, hidden=2048:")
    print("  %-9s %-13s %-10s %-18s" % ("d_expert", "rows/expert", "TFLOPS", "ms (measured band)"))
    for de in (2048, 1024, 512, 256):
        r = expert_ffn(4096, 6, 128, 128, 2048, de)
        print("  %-9d %-13d %-10.1f %.3f - %.3f" % (de, r["rows_per_expert"], r["tflops"],
                                                    r["ms_lo"], r["ms_hi"]))
    print("\nB200 grouped GEMM (this repository), single MoE layer shapes:")
    for e in sorted(B200_GROUPED_TFLOPS):
        r = expert_ffn_b200(4096, 6, e * 8, 8, 4096, 1408)
        print("  %2d local experts: %.0f TFLOPS forward, %.3f ms" % (e, r["tflops"], r["ms"]))
    print("\nCompute is never added to communication here: the two overlap by an amount no")
    print("measurement on hand resolves.")


if __name__ == "__main__":
    main()
