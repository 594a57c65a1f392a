"""Per-device quantities of the cost model: accelerators, the arrival chain, expert memory.

Three questions are answered here, each by one small object.

*What does the device sustain?*  ``Accelerator`` -- HBM bandwidth, capacity, launch time, and the
share of the bandwidth a row gather reaches.  The B200 record comes from this repository's own
measurements (copy bandwidth, bf16 GEMM burst, about 4 us per launch from a graph-free stream);
the Ascend record restates the reference's.

*What does the arrival chain cost?*  The chain (expand pairs, bucket them, gather rows) has a part
that depends only on the number of pairs and a part proportional to the row width.  The
reference's hidden-width sweep (73728 pairs at four widths) is a straight line in the width; its
intercept is the index work (28.6 ns per pair), its slope a gather at about 1.47 TB/s counting a
read and a write.  ``ArrivalChain`` prices any pair count from those two numbers, with a launch
floor.  The fused transport of this repository stores rows at their final position, so on B200
the applicable tier is the one without a chain (``B200_FUSED``).

*How many GPUs must share the experts?*  ``MoEModel`` sizes one expert (weights plus optimizer
state); ``min_expert_parallelism`` returns the smallest power of two that fits a device.

Parity with the reference ``sim/machine.py`` (sweep table :83, decomposition :110-129,
``Accelerator`` :137-175, ``ArrivalChain`` :178-210, ``chain_us_per_row_at`` :226-249, tiers
:252-256, ``MoEModel`` / ``min_expert_parallelism`` / ``spans_multiple_domains`` :264-316).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

from ._text import Column, render_table

BYTES_BF16 = 2

# hidden-width sweep of the arrival chain on the reference machine: width -> ms
CHAIN_H_SWEEP_MS = {1024: 2.37, 2048: 2.51, 4096: 2.85, 8192: 3.79}
CHAIN_H_SWEEP_INPUT_ROWS, CHAIN_H_SWEEP_QUOTA = 24576, 3
CHAIN_H_SWEEP_PAIRS = CHAIN_H_SWEEP_QUOTA * CHAIN_H_SWEEP_INPUT_ROWS
# in-situ calibration point the per-row figures are rebased to
CHAIN_REFERENCE_PAIRS, CHAIN_LEVEL_CALIBRATION_MS = 24576, 1.042
LAUNCH_FLOOR_OPS = 2


def _width_line(points: dict) -> tuple:
    """Least-squares (intercept, slope) of ms against width / 1024."""
    widths = sorted(points)
    u = [w / 1024.0 for w in widths]
    v = [points[w] for w in widths]
    ubar, vbar = math.fsum(u) / len(u), math.fsum(v) / len(v)
    sxy = math.fsum((a - ubar) * (b - vbar) for a, b in zip(u, v))
    sxx = math.fsum((a - ubar) ** 2 for a in u)
    return vbar - sxy / sxx * ubar, sxy / sxx


_fixed, _slope = _width_line(CHAIN_H_SWEEP_MS)
CHAIN_FIXED_MS, CHAIN_PER_1024H_MS = round(_fixed, 4), round(_slope, 4)
INDEX_NS_PER_ROW = 1e6 * CHAIN_FIXED_MS / CHAIN_H_SWEEP_PAIRS
# slope -> bandwidth: every pair reads and writes 1024 elements per 1024 of width
GATHER_GBPS_MEASURED = (2 * BYTES_BF16 * 1024 * CHAIN_H_SWEEP_PAIRS) / (CHAIN_PER_1024H_MS * 1e6)


@dataclass(frozen=True)
class Accelerator:
    name: str
    hbm_gbps: float
    hbm_capacity_gb: float
    launch_ms: float
    gather_eff: float = 0.0
    peak_tflops: float = 0.0
    notes: str = ""

    @classmethod
    def from_gather_bw(cls, name, gather_gbps, hbm_capacity_gb, launch_ms, hbm_gbps=None,
                       peak_tflops=0.0, notes=""):
        """For machines whose sustained gather rate is known directly (the copy rate defaults
        to it, which makes the efficiency 1)."""
        copy_rate = gather_gbps if not hbm_gbps else hbm_gbps
        return cls(name, copy_rate, hbm_capacity_gb, launch_ms, gather_gbps / copy_rate,
                   peak_tflops, notes)

    @property
    def gather_gbps(self) -> float:
        if self.gather_eff > 0.0:
            return self.gather_eff * self.hbm_gbps
        raise ValueError(f"{self.name} has no measured gather efficiency; pass gather_eff or "
                         f"build it with Accelerator.from_gather_bw")

    def usable_bytes(self, reserve_frac: float) -> float:
        return (1.0 - reserve_frac) * self.hbm_capacity_gb * 1e9


B200 = Accelerator("NVIDIA B200", hbm_gbps=6555.8, hbm_capacity_gb=180.0, launch_ms=0.004,
                   gather_eff=0.85, peak_tflops=1639.1,
                   notes="copy bandwidth and bf16 GEMM burst measured on this pool")
ASCEND_910C = Accelerator.from_gather_bw("Ascend 910C die", GATHER_GBPS_MEASURED, 64.0, 0.05,
                                         peak_tflops=376.0, notes="reference measurements")


@dataclass(frozen=True)
class ArrivalChain:
    """``traffic`` counts bytes moved per payload byte (2 = read + write, 1 = a fused kernel that
    writes once, 0 = nothing moves); ``floor_ops`` launches bound the time from below."""
    name: str
    index_ns_per_row: float
    traffic: float = 2.0
    floor_ops: int = LAUNCH_FLOOR_OPS

    def gather_ns_per_row(self, H: int, accel: Accelerator, bytes_per_elem: int = BYTES_BF16):
        moved = self.traffic * bytes_per_elem * H
        return moved / accel.gather_gbps if moved else 0.0

    def ns_per_row(self, H: int, accel: Accelerator, bytes_per_elem: int = BYTES_BF16):
        return self.gather_ns_per_row(H, accel, bytes_per_elem) + self.index_ns_per_row

    def ms(self, rows: int, H: int, accel: Accelerator, bytes_per_elem: int = BYTES_BF16):
        work = 1e-6 * rows * self.ns_per_row(H, accel, bytes_per_elem)
        floor = accel.launch_ms * self.floor_ops
        return work if work > floor else floor

    def us_per_row(self, rows: int, H: int, accel: Accelerator) -> float:
        return 1e3 * self.ms(rows, H, accel) / rows


def chain_us_per_row_at(H: int) -> float:
    """Measured chain cost per pair at hidden width H, rebased onto the in-situ calibration
    (1.042 ms at 24576 pairs, H = 2048).  Only the measured widths are defined."""
    try:
        swept = CHAIN_H_SWEEP_MS[H]
    except KeyError:
        raise ValueError("the hidden-width sweep measured H in %s; widths between them are not "
                         "modelled" % sorted(CHAIN_H_SWEEP_MS)) from None
    scale = CHAIN_LEVEL_CALIBRATION_MS / CHAIN_H_SWEEP_MS[2048]
    return 1e3 * scale * swept / CHAIN_REFERENCE_PAIRS


NO_CHAIN = ArrivalChain("zero implementation overhead", 0.0, traffic=0.0, floor_ops=0)
FUSED_CHAIN = ArrivalChain("fused kernel (K1)", 0.0, traffic=1.0, floor_ops=1)
PYTORCH_CHAIN = ArrivalChain("PyTorch operator chain", INDEX_NS_PER_ROW)
B200_FUSED = NO_CHAIN            # rows are pushed to their final position: nothing to price
TIERS = (PYTORCH_CHAIN, FUSED_CHAIN, NO_CHAIN)


@dataclass(frozen=True)
class MoEModel:
    name: str
    hidden: int
    experts: int
    expert_ffn_mult: float = 4.0
    n_moe_layers: int = 1
    bytes_per_param: int = 2
    optimizer_bytes_per_param: float = 6.0
    matrices_per_expert: int = 3

    @property
    def params_per_expert(self) -> int:
        one_matrix = self.hidden * int(self.expert_ffn_mult * self.hidden)
        return self.n_moe_layers * self.matrices_per_expert * one_matrix

    def bytes_per_expert(self, with_optimizer: bool = True) -> float:
        state = self.optimizer_bytes_per_param if with_optimizer else 0.0
        return (state + self.bytes_per_param) * self.params_per_expert


def _pow2_at_least(v: float) -> int:
    return 1 if v <= 1.0 else 1 << math.ceil(math.log2(v))


def min_expert_parallelism(model: MoEModel, accel: Accelerator, reserve_frac: float,
                           with_optimizer: bool = True) -> int:
    """Smallest power-of-two EP whose expert shard fits the HBM left after ``reserve_frac``
    (never beyond the first power of two that reaches the expert count)."""
    footprint = model.bytes_per_expert(with_optimizer) * model.experts
    ep = _pow2_at_least(model.experts)
    while ep > 1 and footprint / (ep // 2) <= accel.usable_bytes(reserve_frac):
        ep //= 2
    return ep


def spans_multiple_domains(ep: int, domain_size: int) -> bool:
    return domain_size < ep


def report() -> str:
    """Plain-ASCII tables of the accelerator records and the arrival-chain tiers."""
    devices = render_table(
        [Column("device", "%-18s", lambda a: a.name), Column("hbm GB/s", "%9.1f", lambda a: a.hbm_gbps),
         Column("GB", "%6.1f", lambda a: a.hbm_capacity_gb),
         Column("launch us", "%9.1f", lambda a: 1e3 * a.launch_ms)], [B200, ASCEND_910C])
    widths = sorted(CHAIN_H_SWEEP_MS)
    tiers = render_table(
        [Column("H", "%5d", lambda h: h), Column("measured", "%8.2f", CHAIN_H_SWEEP_MS.get)]
        + [Column(t.name.split(" ")[0], "%8.3f",
                  lambda h, t=t: t.ms(CHAIN_H_SWEEP_PAIRS, h, ASCEND_910C)) for t in TIERS], widths)
    tail = "index cost %.1f ns/row, gather %.0f GB/s" % (INDEX_NS_PER_ROW, GATHER_GBPS_MEASURED)
    return "\n".join(["accelerators:", *devices,
                      "arrival chain, %d pairs (ms):" % CHAIN_H_SWEEP_PAIRS, *tiers, tail])


if __name__ == "__main__":
    print(report())
