"""Arrival-chain decomposition and accelerator descriptions.

The arrival chain (expand pairs, bucket sort, gather rows) costs a part that depends only on the
number of pairs (index work) and a part proportional to the row width (the gather).  The
hidden-width sweep of the reference (73728 pairs, H in {1024, 2048, 4096, 8192}) separates the
two by a straight-line fit: 28.6 ns of index work per pair and a row gather running at about
1.47 TB/s.  ``ArrivalChain.ms = max(floor_ops * launch, pairs * (index + H*bytes*traffic/gather))``.
On B200 the fused transport has no chain at all (rows are stored at their final position), which
is the ``B200_FUSED`` tier.

Parity with the reference ``sim/machine.py`` (sweep table :83, decomposition :110-129,
``Accelerator`` :137-175, ``ArrivalChain`` :178-210, ``chain_us_per_row_at`` :226-249, tiers
:252-256, ``MoEModel`` / ``min_expert_parallelism`` / ``spans_multiple_domains`` :264-316).
"""
from __future__ import annotations

from dataclasses import dataclass

BYTES_BF16 = 2
CHAIN_H_SWEEP_MS = {1024: 2.37, 2048: 2.51, 4096: 2.85, 8192: 3.79}
CHAIN_H_SWEEP_INPUT_ROWS = 24576
CHAIN_H_SWEEP_QUOTA = 3
CHAIN_H_SWEEP_PAIRS = CHAIN_H_SWEEP_INPUT_ROWS * CHAIN_H_SWEEP_QUOTA
CHAIN_REFERENCE_PAIRS = 24576
CHAIN_LEVEL_CALIBRATION_MS = 1.042


def _line_fit(table: dict):
    """Ordinary least squares ms = a + b * (H / 1024)."""
    xs = [h / 1024.0 for h in sorted(table)]
    ys = [table[h] for h in sorted(table)]
    n = len(xs)
    mx, my = sum(xs) / n, sum(ys) / n
    slope = sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / sum((x - mx) ** 2 for x in xs)
    return my - slope * mx, slope


CHAIN_FIXED_MS, CHAIN_PER_1024H_MS = (round(v, 4) for v in _line_fit(CHAIN_H_SWEEP_MS))
GATHER_GBPS_MEASURED = (CHAIN_H_SWEEP_PAIRS * 1024 * BYTES_BF16 * 2
                        / (CHAIN_PER_1024H_MS * 1e-3) / 1e9)
INDEX_NS_PER_ROW = CHAIN_FIXED_MS * 1e6 / CHAIN_H_SWEEP_PAIRS
LAUNCH_FLOOR_OPS = 2


@dataclass(frozen=True)
class Accelerator:
    name: str
    hbm_gbps: float
    hbm_capacity_gb: float
    launch_ms: float
    gather_eff: float = 0.0
    peak_tflops: float = 0.0
    notes: str = ""

    @property
    def gather_gbps(self) -> float:
        if self.gather_eff <= 0.0:
            raise ValueError(f"{self.name} has no measured gather efficiency; pass gather_eff or "
                             f"build it with Accelerator.from_gather_bw")
        return self.hbm_gbps * self.gather_eff

    @classmethod
    def from_gather_bw(cls, name, gather_gbps, hbm_capacity_gb, launch_ms, hbm_gbps=None,
                       peak_tflops=0.0, notes=""):
        hbm = hbm_gbps or gather_gbps
        return cls(name=name, hbm_gbps=hbm, hbm_capacity_gb=hbm_capacity_gb, launch_ms=launch_ms,
                   gather_eff=gather_gbps / hbm, peak_tflops=peak_tflops, notes=notes)


# the two machines this repository knows first hand / from the reference
ASCEND_910C = Accelerator.from_gather_bw("Ascend 910C die", GATHER_GBPS_MEASURED, 64.0, 0.05,
                                         peak_tflops=376.0, notes="reference measurements")
B200 = Accelerator("NVIDIA B200", hbm_gbps=6555.8, hbm_capacity_gb=180.0, launch_ms=0.004,
                   gather_eff=0.85, peak_tflops=1639.1,
                   notes="copy bandwidth and bf16 GEMM burst measured on this pool")


@dataclass(frozen=True)
class ArrivalChain:
    name: str
    index_ns_per_row: float
    traffic: float = 2.0          # bytes moved per payload byte (read + write = 2)
    floor_ops: int = LAUNCH_FLOOR_OPS

    def gather_ns_per_row(self, H: int, accel: Accelerator, bytes_per_elem: int = BYTES_BF16):
        if self.traffic == 0.0:
            return 0.0
        return H * bytes_per_elem * self.traffic / accel.gather_gbps

    def ns_per_row(self, H: int, accel: Accelerator, bytes_per_elem: int = BYTES_BF16):
        return self.index_ns_per_row + self.gather_ns_per_row(H, accel, bytes_per_elem)

    def ms(self, rows: int, H: int, accel: Accelerator, bytes_per_elem: int = BYTES_BF16):
        linear = rows * self.ns_per_row(H, accel, bytes_per_elem) / 1e6
        return max(self.floor_ops * accel.launch_ms, linear)

    def us_per_row(self, rows: int, H: int, accel: Accelerator) -> float:
        return self.ms(rows, H, accel) * 1000.0 / rows


def chain_us_per_row_at(H: int) -> float:
    """Measured chain cost per pair at hidden width H, rebased onto the in-situ calibration
    (1.042 ms at 24576 pairs, H = 2048).  Only the measured widths are defined."""
    if H not in CHAIN_H_SWEEP_MS:
        raise ValueError("the hidden-width sweep measured H in %s; widths between them are not "
                         "modelled" % sorted(CHAIN_H_SWEEP_MS))
    rebased = CHAIN_H_SWEEP_MS[H] * CHAIN_LEVEL_CALIBRATION_MS / CHAIN_H_SWEEP_MS[2048]
    return rebased * 1000.0 / CHAIN_REFERENCE_PAIRS


PYTORCH_CHAIN = ArrivalChain("PyTorch operator chain", INDEX_NS_PER_ROW, 2.0)
FUSED_CHAIN = ArrivalChain("fused kernel (K1)", 0.0, 1.0, floor_ops=1)
NO_CHAIN = ArrivalChain("zero implementation overhead", 0.0, 0.0, floor_ops=0)
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
        inter = int(self.hidden * self.expert_ffn_mult)
        return self.matrices_per_expert * self.hidden * inter * self.n_moe_layers

    def bytes_per_expert(self, with_optimizer: bool = True) -> float:
        per = self.bytes_per_param + (self.optimizer_bytes_per_param if with_optimizer else 0.0)
        return self.params_per_expert * per


def min_expert_parallelism(model: MoEModel, accel: Accelerator, reserve_frac: float,
                           with_optimizer: bool = True) -> int:
    """Smallest power-of-two EP whose expert shard fits the HBM left after ``reserve_frac``."""
    usable = accel.hbm_capacity_gb * 1e9 * (1.0 - reserve_frac)
    total = model.experts * model.bytes_per_expert(with_optimizer)
    ep = 1
    while ep < model.experts and total / ep > usable:
        ep *= 2
    return ep


def spans_multiple_domains(ep: int, domain_size: int) -> bool:
    return ep > domain_size


def report() -> str:
    """Plain-ASCII table of the accelerator records and the arrival-chain tiers."""
    out = ["accelerators:"]
    for acc in (ASCEND_910C, B200):
        out.append(f"  {acc.name:<18s} hbm {acc.hbm_gbps:8.1f} GB/s  capacity {acc.hbm_capacity_gb:6.1f} GB"
                   f"  launch {acc.launch_ms * 1e3:5.1f} us")
    out.append(f"arrival chain at the reference point ({CHAIN_REFERENCE_PAIRS} pairs):")
    for H in sorted(CHAIN_H_SWEEP_MS):
        cells = "  ".join(f"{t.name.split(' ')[0]:>8s} {t.ms(CHAIN_H_SWEEP_PAIRS, H, ASCEND_910C):6.3f} ms"
                          for t in TIERS)
        out.append(f"  H={H:<5d} measured {CHAIN_H_SWEEP_MS[H]:5.2f} ms   {cells}")
    out.append(f"index cost {INDEX_NS_PER_ROW:.1f} ns/row, gather {GATHER_GBPS_MEASURED:.0f} GB/s")
    return "\n".join(out)


if __name__ == "__main__":
    print(report())
