"""Scale envelope of a machine: the band of total expert-parameter counts whose MoE layers stay
resident in memory (upper edge) and compute dominated (lower edge).

One ``LayerCost`` prices a single (architecture, machine) pair: the expert matmuls, dispatch +
combine (mirror images, so twice the better of one-hop and two-hop; nothing overlapped), and
the bytes resident per accelerator.  From it,

    utilisation ceiling = GEMM efficiency x compute / (compute + communication)

which bounds what the MoE layers can reach; attention and embeddings are not priced, so it is
not an MFU.  The compute-bound expert width is found by bisection on the same cost.

Public surface of the reference's ``sim/envelope.py`` (``evaluate`` :58-103, ``scale_family`` /
``envelope`` / ``table`` :106-170, ``first_order_threshold`` / ``compute_bound_threshold``
:173-231).
"""
from __future__ import annotations

from dataclasses import dataclass, replace

from . import codesign as cd
from ._text import Column, render_table
from .codesign import UNMEASURED, Machine, MemoryProfile, MoEArch

DEFAULT_FACTORS = (0.125, 0.25, 0.5, 1, 2, 4, 8, 16, 32)
GIB = float(1 << 30)


@dataclass(frozen=True)
class Point:
    arch: MoEArch
    total_params: float
    active_params: float
    params_per_accel: float
    fits: bool
    resident_gib_per_accel: float
    compute_ms: float
    comm_ms: float
    strategy: str
    gemm_efficiency: float
    compute_share: float
    utilisation_ceiling: float
    rows_per_expert: int
    expert_bound_by: str


def _params(arch: MoEArch, experts_counted: int) -> float:
    return (experts_counted + arch.n_shared_experts) * arch.n_moe_layers * arch.params_per_expert()


def total_params(arch: MoEArch) -> float:
    return _params(arch, arch.n_experts)


def active_params(arch: MoEArch) -> float:
    return _params(arch, arch.k)


class LayerCost:
    """Expert compute, dispatch + combine and residency of one architecture on one machine."""

    def __init__(self, arch: MoEArch, machine: Machine, mem: MemoryProfile = UNMEASURED,
                 strategy: str = "best"):
        self.arch, self.machine, self.ep = arch, machine, machine.fabric.ep
        self.matmul = cd.expert_matmul(arch, machine, self.ep)
        self.hops = cd.dispatch_breakdown(arch, machine)
        self.mem = mem
        self.strategy = self._choose(strategy)

    def _choose(self, wanted: str) -> str:
        if wanted in ("one-hop", "two-hop"):
            return wanted
        h = self.hops
        applies = h["domain_condition"] and h["fanout_condition"]
        return "two-hop" if applies and h["two_hop_ms"] < h["one_hop_ms"] else "one-hop"

    @property
    def compute_ms(self) -> float:
        return self.matmul["ms"]

    @property
    def comm_ms(self) -> float:          # there and back
        return 2.0 * self.hops["two_hop_ms" if self.strategy == "two-hop" else "one_hop_ms"]

    @property
    def compute_share(self) -> float:
        whole = self.compute_ms + self.comm_ms
        return self.compute_ms / whole if whole > 0 else 0.0

    @property
    def gemm_efficiency(self) -> float:
        t = self.matmul["ms_compute_bound"]
        peak = self.machine.peak_tflops
        if t <= 0 or not peak:
            return 0.0
        return self.matmul["flops"] / (t * 1e-3) / 1e12 / peak

    @property
    def compute_bound(self) -> bool:
        return self.compute_ms >= self.comm_ms

    def point(self) -> Point:
        res = cd.residency(self.arch, self.machine, self.ep, self.mem)
        tot, eff, share = total_params(self.arch), self.gemm_efficiency, self.compute_share
        return Point(self.arch, tot, active_params(self.arch), tot / self.ep, res["fits"],
                     res["total_bytes"] / GIB, self.compute_ms, self.comm_ms, self.strategy, eff,
                     share, eff * share, self.matmul["rows_per_expert"], self.matmul["bound_by"])


def evaluate(arch: MoEArch, machine: Machine, mem: MemoryProfile = UNMEASURED) -> Point:
    return LayerCost(arch, machine, mem).point()


def scale_family(base: MoEArch, factors) -> list:
    counts = (int(round(base.n_experts * f)) for f in factors)
    return [replace(base, name="%s-E%d" % (base.name, n), n_experts=n) for n in counts
            if n >= base.k]


def envelope(base: MoEArch, machine: Machine, factors=DEFAULT_FACTORS, floor: float = 0.5,
             mem: MemoryProfile = UNMEASURED) -> dict:
    points = [evaluate(arch, machine, mem) for arch in scale_family(base, factors)]
    inside = sorted(p.total_params for p in points if p.fits and p.compute_share >= floor)
    band = (inside[0], inside[-1]) if inside else (None, None)
    return {
        "points": points, "band": band, "floor": floor, "accelerators": machine.fabric.ep,
        "residency_measured": mem.measured,
        "upper_edge": "expert residency exceeds usable memory per accelerator",
        "lower_edge": "compute share falls below %.0f%%, so the moe layer is communication bound "
                      "whatever overlaps" % (100 * floor),
        "caveat": "mixture-of-experts layers only; attention and embeddings are not priced, so "
                  "this is not an end-to-end MFU",
    }


def _state(p: Point, floor: float) -> str:
    if not p.fits:
        return "does not fit"
    return "ok" if p.compute_share >= floor else "comm bound"


def table(env: dict) -> str:
    columns = (
        Column("experts", "%-9d", lambda p: p.arch.n_experts),
        Column("total P", "%12.3g", lambda p: p.total_params),
        Column("P/accel", "%12.3g", lambda p: p.params_per_accel),
        Column("rows/exp", "%10d", lambda p: p.rows_per_expert),
        Column("compute", "%9.3f", lambda p: p.compute_ms),
        Column("comm", "%9.3f", lambda p: p.comm_ms),
        Column("ceiling", "%8.1f%%", lambda p: 100 * p.utilisation_ceiling, head="%9s"),
        Column("state", "%-9s", lambda p: _state(p, env["floor"])),
    )
    edges = ["%.3g" % v if v else "none" for v in env["band"]]
    tail = ["", "band on %d accelerators: %s to %s total expert parameters"
            % (env["accelerators"], edges[0], edges[1]),
            "upper edge: " + env["upper_edge"], "lower edge: " + env["lower_edge"], env["caveat"]]
    return "\n".join(render_table(columns, env["points"], rule=88) + tail)


def first_order_threshold(machine) -> float:
    """Expert width at which compute and slow-side bytes balance to first order: each token row
    costs 3 matmuls of 2 * H * d FLOPs and crosses the slow level as 2 * H bytes."""
    flops_per_s = machine.peak_tflops * 1e12
    slow_bytes_per_s = machine.fabric.beta_inter_gbps * 1e9
    return flops_per_s / (3.0 * slow_bytes_per_s)


def _first_true(lo: int, hi: int, pred) -> int:
    """Smallest integer in [lo, hi] satisfying a monotone predicate, or -1 when none does."""
    if pred(lo):
        return lo
    if not pred(hi):
        return -1
    while hi - lo > 1:
        mid = (lo + hi) >> 1
        lo, hi = (lo, mid) if pred(mid) else (mid, hi)
    return hi


def compute_bound_threshold(template: MoEArch, machine: Machine, strategy: str = "best",
                            lo: int = 128, hi: int = 262144) -> int:
    """Smallest expert width whose matmul time is at least dispatch + combine (-1: none)."""
    def wide_enough(width: int) -> bool:
        return LayerCost(replace(template, d_expert=int(width)), machine,
                         strategy=strategy).compute_bound
    return _first_true(lo, hi, wide_enough)


def main() -> None:
    for m in (cd.synthetic_dgx_h100(), cd.hgx_b200()):
        print("Envelope on the %s (sensitivity; residency unmeasured)" % m.fabric.name)
        print()
        print(table(envelope(cd.REFERENCE_ARCH, m)))
        print()
        print("first-order compute/comm balance width: %d" % first_order_threshold(m))
        print("full-model compute-bound width, best strategy: %d"
              % compute_bound_threshold(cd.REFERENCE_ARCH, m))
        print()


if __name__ == "__main__":
    main()
