"""Expert-FFN compute priced from measured GEMM throughput.

A ``ThroughputCurve`` is a measured (size, TFLOPS) table read by clamped linear interpolation.
Two are registered: the reference platform's square bf16 GEMMs (Ascend 910C), with eight
non-square expert shapes that settled how a (rows, hidden, expert width) problem is indexed
into it -- by the geometric mean of the three dimensions, 6.4 % median error -- and this
repository's tcgen05 grouped GEMM on a B200, indexed by the number of local experts (few long
groups run on CTA pairs, many short ones pay tile padding).  ``expert_ffn`` / ``expert_ffn_b200``
price the routed experts of one rank and one layer.  Compute is never added to communication
here: how much of the two overlaps is a property of the schedule, not of this table.

Public surface of the reference's ``sim/compute.py`` (tables :65-84, ``achieved_tflops`` /
``index_dims`` / ``efficiency_bracket`` :103-139, ``expert_ffn`` :142-178,
``comm_share_upper_bound`` :181-190).
"""
from __future__ import annotations

from bisect import bisect_right

from .records import GEMM_TFLOPS, INDEX_RULE_ERROR, NONSQUARE_TFLOPS


class ThroughputCurve:
    """Measured ``(x, TFLOPS)`` points; values between points are interpolated linearly and
    values outside the measured range take the nearest end point."""

    def __init__(self, points):
        self.points = sorted((float(x), float(y)) for x, y in points)
        self.xs = [x for x, _ in self.points]

    def __call__(self, x: float) -> float:
        pts, xs = self.points, self.xs
        x = min(max(float(x), xs[0]), xs[-1])
        hi = min(bisect_right(xs, x), len(xs) - 1)
        (x0, y0), (x1, y1) = pts[hi - 1] if hi else pts[0], pts[hi]
        return y1 if x1 == x0 else y0 + (y1 - y0) * (x - x0) / (x1 - x0)

    @property
    def peak(self) -> float:
        return max(y for _, y in self.points)


PLATFORM_A_SQUARE = ThroughputCurve(GEMM_TFLOPS)
PEAK_TFLOPS = PLATFORM_A_SQUARE.peak

# candidate ways to turn a (rows, hidden, d_expert) problem into one curve index
_RULES = {
    "min_dim": lambda r, h, d: float(min(r, h, d)),
    "geometric_mean": lambda r, h, d: (r * h * d) ** (1.0 / 3.0),
    "rows": lambda r, h, d: float(r),
}
INDEX_RULES = tuple(_RULES)
INDEX_RULE = "geometric_mean"

# B200, this repository's grouped GEMM (24576 rows, d_model 4096, expert width 1408), TFLOPS by
# number of local experts; cuBLAS 8192^3 on the same GPU for scale.
B200_GROUPED_TFLOPS = {
    8: {"fwd_swiglu": 1258.9, "fwd": 1306.8, "gemm2": 1186.8, "dgrad": 1301.4, "wgrad": 1259.6},
    64: {"fwd_swiglu": 1034.2, "fwd": 1071.1, "gemm2": 992.0, "dgrad": 1026.3, "wgrad": 738.1},
}
B200_CUBLAS_8192_TFLOPS = 1604.8
# FLOP-weighted mix of the kernels in one pass: forward = gate + up (SwiGLU GEMM) + down;
# a training step adds one dgrad and one wgrad per matrix
_B200_MIX = {
    False: {"fwd_swiglu": 2, "gemm2": 1},
    True: {"fwd_swiglu": 2, "gemm2": 1, "dgrad": 3, "wgrad": 3},
}


def _b200_curve(training: bool) -> ThroughputCurve:
    mix = _B200_MIX[training]
    weight = float(sum(mix.values()))
    return ThroughputCurve((experts, sum(v[name] * n for name, n in mix.items()) / weight)
                           for experts, v in B200_GROUPED_TFLOPS.items())


def achieved_tflops(dim: float, table=None) -> float:
    return (ThroughputCurve(table) if table else PLATFORM_A_SQUARE)(dim)


def index_dims(rows: int, hidden: int, d_expert: int) -> dict:
    return {name: rule(rows, hidden, d_expert) for name, rule in _RULES.items()}


def efficiency_bracket(rows: int, hidden: int, d_expert: int) -> dict:
    per_rule = {name: PLATFORM_A_SQUARE(x) for name, x in index_dims(rows, hidden, d_expert).items()}
    ordered = sorted(per_rule.values())
    return {"per_rule": per_rule, "lo": ordered[0], "hi": ordered[-1],
            "spread": ordered[-1] / ordered[0]}


def _local_shape(tokens_per_rank: int, k: int, n_experts: int, ep: int):
    """(local experts, rows per local expert) under balanced routing, each at least one."""
    local = n_experts // ep or 1
    return local, tokens_per_rank * k // local or 1


def _ms(flops: float, tflops: float) -> float:
    return flops / (tflops * 1e9)


def expert_ffn(tokens_per_rank: int, k: int, n_experts: int, ep: int, hidden: int,
               d_expert: int, n_mats: int = 2, backward: bool = False) -> dict:
    """Exact FLOPs of the routed experts of one rank and their time on platform A."""
    local, rows = _local_shape(tokens_per_rank, k, n_experts, ep)
    passes = 2.0 if backward else 1.0
    flops = 2.0 * rows * hidden * d_expert * n_mats * local * passes
    bracket = efficiency_bracket(rows, hidden, d_expert)
    rate = bracket["per_rule"][INDEX_RULE]
    centre, worst = _ms(flops, rate), INDEX_RULE_ERROR["worst"]
    return {
        "flops": flops, "rows_per_expert": rows, "experts_local": local, "tflops": rate,
        "ms": centre, "ms_lo": centre * (1.0 - worst), "ms_hi": centre * (1.0 + worst),
        "rule": INDEX_RULE, "rule_error": dict(INDEX_RULE_ERROR),
        "ms_fast": _ms(flops, bracket["hi"]), "ms_slow": _ms(flops, bracket["lo"]),
        "tflops_bracket": (bracket["lo"], bracket["hi"]), "assumption_spread": bracket["spread"],
        "efficiency_vs_peak": rate / PEAK_TFLOPS,
    }


def expert_ffn_b200(tokens_per_rank: int, k: int, n_experts: int, ep: int, hidden: int,
                    d_expert: int, backward: bool = False) -> dict:
    """Same ledger priced with the B200 grouped-GEMM measurements (three matrices: gate, up,
    down); throughput interpolated in the number of local experts."""
    local, _ = _local_shape(tokens_per_rank, k, n_experts, ep)
    flops = 2.0 * tokens_per_rank * k * hidden * d_expert * 3 * (3.0 if backward else 1.0)
    rate = _b200_curve(bool(backward))(local)
    return {"flops": flops, "experts_local": local, "tflops": rate, "ms": _ms(flops, rate)}


def comm_share_upper_bound(comm_ms: float, compute_ms: float) -> float:
    whole = comm_ms + compute_ms
    return float("nan") if whole <= 0 else comm_ms / whole


def report() -> list:
    out = ["Measured bf16 GEMM roofline, platform A (256 samples per size):"]
    out += ["  %6d  %6.1f TFLOPS  %3.0f%% of peak" % (n, t, 100 * t / PEAK_TFLOPS)
            for n, t in GEMM_TFLOPS]
    out += ["", "Measured expert-FFN shapes, and what each index rule would have said:",
            "  %-22s %9s %8s %8s %8s" % ("rows x hidden x d_exp", "measured", "geo-mean",
                                         "min-dim", "rows")]
    for shape in sorted(NONSQUARE_TFLOPS):
        said = efficiency_bracket(*shape)["per_rule"]
        out.append("  %-22s %9.1f %8.0f %8.0f %8.0f"
                   % ("%d x %d x %d" % shape, NONSQUARE_TFLOPS[shape], said["geometric_mean"],
                      said["min_dim"], said["rows"]))
    out += ["  geometric mean is the rule in use: %.1f%% median error, worst %.1f%%"
            % (100 * INDEX_RULE_ERROR["median_abs"], 100 * INDEX_RULE_ERROR["worst"]),
            "", "Expert-FFN forward, one layer, one rank: T=4096, k=6, E=128, EP=128, hidden=2048:",
            "  %-9s %-13s %-10s %-18s" % ("d_expert", "rows/expert", "TFLOPS",
                                          "ms (measured band)")]
    for width in (2048, 1024, 512, 256):
        r = expert_ffn(4096, 6, 128, 128, 2048, width)
        out.append("  %-9d %-13d %-10.1f %.3f - %.3f"
                   % (width, r["rows_per_expert"], r["tflops"], r["ms_lo"], r["ms_hi"]))
    out += ["", "B200 grouped GEMM (this repository), single MoE layer shapes:"]
    for local in sorted(B200_GROUPED_TFLOPS):
        r = expert_ffn_b200(4096, 6, local * 8, 8, 4096, 1408)
        out.append("  %2d local experts: %.0f TFLOPS forward, %.3f ms" % (local, r["tflops"], r["ms"]))
    out += ["", "Compute is never added to communication here: the two overlap by an amount no",
            "measurement on hand resolves."]
    return out


def main() -> None:
    print("\n".join(report()))


if __name__ == "__main__":
    main()
