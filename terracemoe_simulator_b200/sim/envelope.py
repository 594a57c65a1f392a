"""Scale envelope: for which total expert-parameter counts does a machine keep the MoE layers
both resident and compute dominated?

``utilisation ceiling = GEMM efficiency x compute / (compute + 2 x dispatch)`` (dispatch and
combine mirror each other, the better of one-hop and two-hop is taken, nothing is assumed to
overlap).  The upper edge of the band is memory residency, the lower edge a compute share below
``floor``.  MoE layers only: attention and embeddings are not priced, so this is not an MFU.

Parity with the reference ``sim/envelope.py`` (``evaluate`` :58-103, ``scale_family`` /
``envelope`` / ``table`` :106-170, ``first_order_threshold`` / ``compute_bound_threshold``
:173-231).
"""
from __future__ import annotations

from dataclasses import dataclass, replace

from .codesign import (UNMEASURED, Machine, MemoryProfile, MoEArch, dispatch_breakdown,
                       expert_matmul, residency)


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


def total_params(arch: MoEArch) -> float:
    return (arch.n_experts + arch.n_shared_experts) * arch.n_moe_layers * arch.params_per_expert()


def active_params(arch: MoEArch) -> float:
    return (arch.k + arch.n_shared_experts) * arch.n_moe_layers * arch.params_per_expert()


def _best_dispatch(d: dict):
    if d["domain_condition"] and d["fanout_condition"] and d["two_hop_ms"] < d["one_hop_ms"]:
        return d["two_hop_ms"], "two-hop"
    return d["one_hop_ms"], "one-hop"


def evaluate(arch: MoEArch, machine: Machine, mem: MemoryProfile = UNMEASURED) -> Point:
    ep = machine.fabric.ep
    mm = expert_matmul(arch, machine, ep)
    comm, strategy = _best_dispatch(dispatch_breakdown(arch, machine))
    comm *= 2.0
    res = residency(arch, machine, ep, mem)
    achieved = mm["flops"] / (mm["ms_compute_bound"] * 1e-3) / 1e12 if mm["ms_compute_bound"] > 0 \
        else 0.0
    eff = achieved / machine.peak_tflops if machine.peak_tflops else 0.0
    share = mm["ms"] / (mm["ms"] + comm) if mm["ms"] + comm > 0 else 0.0
    tot = total_params(arch)
    return Point(arch=arch, total_params=tot, active_params=active_params(arch),
                 params_per_accel=tot / ep, fits=res["fits"],
                 resident_gib_per_accel=res["total_bytes"] / 2 ** 30, compute_ms=mm["ms"],
                 comm_ms=comm, strategy=strategy, gemm_efficiency=eff, compute_share=share,
                 utilisation_ceiling=eff * share, rows_per_expert=mm["rows_per_expert"],
                 expert_bound_by=mm["bound_by"])


def scale_family(base: MoEArch, factors) -> list:
    out = []
    for f in factors:
        E = int(round(base.n_experts * f))
        if E >= base.k:
            out.append(replace(base, name="%s-E%d" % (base.name, E), n_experts=E))
    return out


def envelope(base: MoEArch, machine: Machine, factors=(0.125, 0.25, 0.5, 1, 2, 4, 8, 16, 32),
             floor: float = 0.5, mem: MemoryProfile = UNMEASURED) -> dict:
    pts = [evaluate(a, machine, mem) for a in scale_family(base, factors)]
    ok = [p.total_params for p in pts if p.fits and p.compute_share >= floor]
    return {"points": pts, "band": (min(ok, default=None), max(ok, default=None)),
            "upper_edge": "expert residency exceeds usable memory per accelerator",
            "lower_edge": "compute share falls below %.0f%%, so the moe layer is communication "
                          "bound whatever overlaps" % (100 * floor),
            "floor": floor, "accelerators": machine.fabric.ep,
            "caveat": "mixture-of-experts layers only; attention and embeddings are not priced, "
                      "so this is not an end-to-end MFU",
            "residency_measured": mem.measured}


def table(env: dict) -> str:
    lines = ["%-9s %12s %12s %10s %9s %9s %9s %-9s" % ("experts", "total P", "P/accel",
                                                       "rows/exp", "compute", "comm", "ceiling",
                                                       "state"), "-" * 88]
    for p in env["points"]:
        state = "does not fit" if not p.fits else \
            "comm bound" if p.compute_share < env["floor"] else "ok"
        lines.append("%-9d %12.3g %12.3g %10d %9.3f %9.3f %8.1f%% %-9s"
                     % (p.arch.n_experts, p.total_params, p.params_per_accel, p.rows_per_expert,
                        p.compute_ms, p.comm_ms, 100 * p.utilisation_ceiling, state))
    lo, hi = env["band"]
    lines += ["", "band on %d accelerators: %s to %s total expert parameters"
              % (env["accelerators"], "%.3g" % lo if lo else "none", "%.3g" % hi if hi else "none"),
              "upper edge: " + env["upper_edge"], "lower edge: " + env["lower_edge"],
              env["caveat"]]
    return "\n".join(lines)


def first_order_threshold(machine) -> float:
    """Expert width at which compute and slow-side bytes balance to first order."""
    return machine.peak_tflops * 1e12 / (3.0 * machine.fabric.beta_inter_gbps * 1e9)


def compute_bound_threshold(template: MoEArch, machine: Machine, strategy: str = "best",
                            lo: int = 128, hi: int = 262144) -> int:
    """Smallest expert width whose matmul time is at least dispatch + combine (-1: none)."""
    def bound(d):
        a = replace(template, d_expert=int(d))
        mm = expert_matmul(a, machine, machine.fabric.ep)
        br = dispatch_breakdown(a, machine)
        if strategy == "one-hop":
            comm = br["one_hop_ms"]
        elif strategy == "two-hop":
            comm = br["two_hop_ms"]
        elif br["domain_condition"] and br["fanout_condition"]:
            comm = min(br["one_hop_ms"], br["two_hop_ms"])
        else:
            comm = br["one_hop_ms"]
        return mm["ms"] >= 2.0 * comm
    if bound(lo):
        return lo
    if not bound(hi):
        return -1
    while lo + 1 < hi:
        mid = (lo + hi) // 2
        if bound(mid):
            hi = mid
        else:
            lo = mid
    return hi


def main() -> None:
    from .codesign import REFERENCE_ARCH, hgx_b200, synthetic_dgx_h100
    for m in (synthetic_dgx_h100(), hgx_b200()):
        print("Envelope on the %s (sensitivity; residency unmeasured)" % m.fabric.name)
        print()
        print(table(envelope(REFERENCE_ARCH, m)))
        print()
        print("first-order compute/comm balance width: %d" % first_order_threshold(m))
        print("full-model compute-bound width, best strategy: %d"
              % compute_bound_threshold(REFERENCE_ARCH, m))
        print()


if __name__ == "__main__":
    main()
