"""Co-design layer: an MoE architecture on a machine (accelerator + fabric + arrival-chain tier).

For one (architecture, machine) pair it reports what binds first -- expert memory residency, the
expert matmuls (compute or memory bound), or the dispatch -- as separate per-call / per-layer
terms.  They are deliberately NOT added into a step time: the step-level gate of the model fails.

Parity with the reference ``sim/codesign.py``: ``MoEArch`` / ``Fabric`` / ``Machine`` :56-173,
``expert_matmul`` :180-222, ``MemoryProfile`` / ``UNMEASURED`` / ``residency`` /
``min_ep_for_memory`` :229-317, ``dispatch_breakdown`` :324-361, ``profile`` / ``sweep``
:364-401, ``synthetic_dgx_h100`` :408-438, ``REFERENCE_ARCH`` / ``m_table`` :442-460.
New: ``hgx_b200`` (the machine this repository measures on).
"""
from __future__ import annotations

from dataclasses import dataclass, replace

from .compute import INDEX_RULE, INDEX_RULE_ERROR, PEAK_TFLOPS, efficiency_bracket
from .core import ClusterSpec, Level, MoEGeometry, one_hop_call, two_hop_call
from .machine import Accelerator, ArrivalChain, PYTORCH_CHAIN


@dataclass(frozen=True)
class MoEArch:
    name: str
    hidden: int
    d_expert: int
    n_experts: int
    k: int
    M: int = 1
    n_shared_experts: int = 0
    n_moe_layers: int = 1
    seq: int = 4096
    mbs: int = 1
    gbs: int = 512
    n_mats: int = 3
    bytes_per_elem: int = 2
    optimizer_bytes_per_param: float = 6.0

    @property
    def q(self) -> int:
        if self.k % self.M:
            raise ValueError("%s: k=%d is not divisible by M=%d, so the per-group quota k/M is "
                             "not an integer" % (self.name, self.k, self.M))
        return self.k // self.M

    @property
    def tokens_per_rank(self) -> int:
        return self.seq * self.mbs

    def params_per_expert(self) -> int:
        return self.n_mats * self.hidden * self.d_expert

    def expert_bytes_all_layers(self, with_optimizer: bool = True) -> float:
        per = self.bytes_per_elem + (self.optimizer_bytes_per_param if with_optimizer else 0.0)
        return ((self.n_experts + self.n_shared_experts) * self.n_moe_layers
                * self.params_per_expert() * per)


@dataclass(frozen=True)
class Fabric:
    name: str
    cards_per_node: int
    nodes: int
    beta_intra_gbps: float
    beta_inter_gbps: float
    alpha_ms: tuple                     # ((world, ms), ...)
    x_half_bytes: float = 0.0

    @property
    def ep(self) -> int:
        return self.cards_per_node * self.nodes

    @property
    def ratio(self) -> float:
        return self.beta_intra_gbps / self.beta_inter_gbps

    def alpha_at(self, world: int) -> float:
        pts = sorted(self.alpha_ms)
        if world <= pts[0][0]:
            return pts[0][1]
        if world >= pts[-1][0]:
            return pts[-1][1]
        for (w0, a0), (w1, a1) in zip(pts, pts[1:]):
            if w0 <= world <= w1:
                return a0 + (a1 - a0) * (world - w0) / float(w1 - w0)
        return pts[-1][1]

    def fixed_cost_condition(self) -> dict:
        two = self.alpha_at(self.nodes) + self.alpha_at(self.cards_per_node)
        one = self.alpha_at(self.ep)
        return {"two_hop_alpha_ms": two, "one_hop_alpha_ms": one, "clears": two < one,
                "margin_ms": one - two}


@dataclass(frozen=True)
class Machine:
    accel: Accelerator
    fabric: Fabric
    chain: ArrivalChain = PYTORCH_CHAIN

    @property
    def peak_tflops(self) -> float:
        return self.accel.peak_tflops or PEAK_TFLOPS

    @property
    def balance_flops_per_byte(self) -> float:
        return self.peak_tflops * 1e12 / (self.accel.hbm_gbps * 1e9)

    @property
    def transfers_compute(self) -> bool:
        return bool(self.accel.peak_tflops)


def expert_matmul(arch: MoEArch, machine: Machine, ep: int, backward: bool = False) -> dict:
    """Routed experts of one rank and one layer: the slower of a compute-bound time (measured
    GEMM efficiency curve, rescaled to the machine's peak) and a memory-bound time (weights plus
    activations once through HBM)."""
    local = max(arch.n_experts // ep, 1)
    rows = max(arch.tokens_per_rank * arch.k // local, 1)
    passes = 2.0 if backward else 1.0
    flops = 2.0 * rows * arch.hidden * arch.d_expert * arch.n_mats * local * passes
    tflops = efficiency_bracket(rows, arch.hidden, arch.d_expert)["per_rule"][INDEX_RULE]
    if machine.accel.peak_tflops:
        tflops *= machine.accel.peak_tflops / PEAK_TFLOPS
    ms_compute = flops / (tflops * 1e12) * 1e3
    weight_bytes = local * arch.params_per_expert() * arch.bytes_per_elem * passes
    act_bytes = rows * local * (arch.hidden + 2.0 * arch.d_expert) * arch.bytes_per_elem
    ms_memory = (weight_bytes + act_bytes) / (machine.accel.hbm_gbps * 1e9) * 1e3
    return {"rows_per_expert": rows, "experts_local": local, "flops": flops,
            "ms_compute_bound": ms_compute, "ms_memory_bound": ms_memory,
            "ms": max(ms_compute, ms_memory),
            "bound_by": "memory" if ms_memory > ms_compute else "compute",
            "arithmetic_intensity": rows, "machine_balance": machine.balance_flops_per_byte,
            "compute_measured": rows >= 1536 and not machine.accel.peak_tflops,
            "roofline_borrowed": not machine.transfers_compute, "tflops_rule": INDEX_RULE,
            "tflops_worst_error": INDEX_RULE_ERROR["worst"]}


@dataclass(frozen=True)
class MemoryProfile:
    name: str
    activation_bytes_per_token_layer: float
    overhead_frac: float
    recompute: str = "unknown"
    measured: bool = False
    source: str = ""


UNMEASURED = MemoryProfile(name="unmeasured placeholder", activation_bytes_per_token_layer=0.0,
                           overhead_frac=0.15, recompute="assumed full recompute", measured=False,
                           source="invented; a residency measurement protocol would replace it")


def residency(arch: MoEArch, machine: Machine, ep: int, profile: MemoryProfile = UNMEASURED,
              non_expert_params: int = 0) -> dict:
    expert = arch.expert_bytes_all_layers(with_optimizer=True) / ep
    non_expert = non_expert_params * (arch.bytes_per_elem + arch.optimizer_bytes_per_param)
    act = profile.activation_bytes_per_token_layer * arch.tokens_per_rank * arch.n_moe_layers
    cap = machine.accel.hbm_capacity_gb * 1e9
    overhead = cap * profile.overhead_frac
    total = expert + non_expert + act + overhead
    tag = ("measured: " if profile.measured else "ASSUMED: ") + profile.source
    return {"expert_bytes": expert, "non_expert_bytes": non_expert, "activation_bytes": act,
            "overhead_bytes": overhead, "total_bytes": total, "capacity_bytes": cap,
            "fits": total <= cap, "headroom_bytes": cap - total,
            "provenance": {
                "expert_bytes": "computed from the architecture and the optimizer",
                "non_expert_bytes": "computed" if non_expert_params else
                "NOT SUPPLIED: attention and embeddings omitted",
                "activation_bytes": tag, "overhead_bytes": tag},
            "measured": profile.measured, "profile": profile.name}


def min_ep_for_memory(arch: MoEArch, machine: Machine, profile: MemoryProfile = UNMEASURED,
                      non_expert_params: int = 0) -> dict:
    ep = 1
    while ep < arch.n_experts:
        r = residency(arch, machine, ep, profile, non_expert_params)
        if r["fits"]:
            return {"min_ep": ep, "residency": r, "measured": r["measured"]}
        ep *= 2
    r = residency(arch, machine, arch.n_experts, profile, non_expert_params)
    return {"min_ep": arch.n_experts if r["fits"] else -1, "residency": r,
            "measured": r["measured"]}


def dispatch_breakdown(arch: MoEArch, machine: Machine) -> dict:
    from .calibrate import saturating_beta
    f = machine.fabric
    pairs = arch.tokens_per_rank * arch.k
    chain_ms = machine.chain.ms(pairs, arch.hidden, machine.accel)
    alpha = sorted(f.alpha_ms)
    slow = saturating_beta(f.beta_inter_gbps, f.x_half_bytes)
    cluster = ClusterSpec(
        name=f.name, R=f.cards_per_node,
        fast=Level("fast", alpha, saturating_beta(f.beta_intra_gbps, f.x_half_bytes)),
        slow=Level("slow", alpha, slow), flat=Level("flat", alpha, slow),
        chain_us_per_row=chain_ms * 1000.0 / pairs)
    g = MoEGeometry(name=arch.name, n_groups=f.nodes, R=f.cards_per_node, k=arch.k, M=arch.M,
                    H=arch.hidden, seq=arch.seq, mbs=arch.mbs, gbs=arch.gbs,
                    moe_layers=arch.n_moe_layers, bytes_per_elem=arch.bytes_per_elem)
    one, two = one_hop_call(cluster, g), two_hop_call(cluster, g)
    return {"ep": f.ep, "q": arch.q, "ratio": f.ratio, "one_hop_ms": one, "two_hop_ms": two,
            "G": one / two, "chain_us_per_row": chain_ms * 1000.0 / pairs, "chain_ms": chain_ms,
            "chain_share_of_two_hop": chain_ms / two, "domain_condition": f.ep > f.cards_per_node,
            "fanout_condition": arch.q >= 2}


def profile(arch: MoEArch, machine: Machine, mem: MemoryProfile = UNMEASURED,
            non_expert_params: int = 0) -> dict:
    mep = min_ep_for_memory(arch, machine, mem, non_expert_params)
    floor = mep["min_ep"]
    fits = 0 < floor <= machine.fabric.ep
    mm = expert_matmul(arch, machine, machine.fabric.ep)
    if not fits:
        binds = "memory capacity"
    elif mm["bound_by"] == "memory":
        binds = "expert matmul, memory bound"
    else:
        binds = "expert matmul, compute bound"
    return {"arch": arch.name, "machine": machine.fabric.name,
            "memory": {"min_ep": floor, "configured_ep": machine.fabric.ep, "fits": fits,
                       "measured": mep["measured"], "breakdown": mep["residency"],
                       "expert_gib": arch.expert_bytes_all_layers() / 2 ** 30},
            "expert_matmul": mm, "dispatch": dispatch_breakdown(arch, machine), "binds": binds,
            "caveat": "step-level composition is behind a failing gate; the terms above are "
                      "per-call and per-layer and do not add to a step time",
            "memory_caveat": None if mep["measured"] else
            "the residency verdict rests on an unmeasured memory profile (docs/11-residency.md lists "
            "what has to be measured)"}


def sweep(base: MoEArch, machine: Machine, knob: str, values, mem: MemoryProfile = UNMEASURED):
    out = []
    for v in values:
        try:
            out.append((v, profile(replace(base, **{knob: v}), machine, mem)))
        except ValueError as exc:
            out.append((v, {"error": str(exc)}))
    return out


def synthetic_dgx_h100(nodes: int = 16, chain: ArrivalChain = PYTORCH_CHAIN) -> Machine:
    """Datasheet H100 nodes behind NDR400; gather and launch constants borrowed from platform A."""
    from .calibrate import ALPHA_PTS, X_HALF_FLAT
    from .machine import GATHER_GBPS_MEASURED
    accel = Accelerator.from_gather_bw(
        "synthetic H100 SXM", gather_gbps=GATHER_GBPS_MEASURED, hbm_capacity_gb=80.0,
        launch_ms=0.129, hbm_gbps=3350.0, peak_tflops=989.0,
        notes="vendor datasheet numbers; gather and launch borrowed from platform A")
    fabric = Fabric(name="synthetic DGX H100 + NDR400, %d nodes" % nodes, cards_per_node=8,
                    nodes=nodes, beta_intra_gbps=450.0, beta_inter_gbps=50.0,
                    alpha_ms=tuple(ALPHA_PTS), x_half_bytes=float(X_HALF_FLAT))
    return Machine(accel, fabric, chain)


def hgx_b200(group_size: int = 2, chain: ArrivalChain | None = None) -> Machine:
    """One 8 x B200 box: a single NVSwitch domain split into logical groups of ``group_size``."""
    from . import calibrate as cal
    from .machine import B200, B200_FUSED
    a = cal.B200_ALPHA_US["flat"] / 1000.0
    fabric = Fabric(name="HGX B200, %d logical groups of %d" % (8 // group_size, group_size),
                    cards_per_node=group_size, nodes=8 // group_size,
                    beta_intra_gbps=cal.B200_BETA_GBPS, beta_inter_gbps=cal.B200_BETA_GBPS,
                    alpha_ms=((2, a), (16, a)), x_half_bytes=float(cal.B200_X_HALF))
    return Machine(B200, fabric, chain or B200_FUSED)


REFERENCE_ARCH = MoEArch(name="reference", hidden=7168, d_expert=2048, n_experts=256, k=8, M=4,
                         n_moe_layers=1, seq=4096, mbs=1)


def m_table(arch: MoEArch = REFERENCE_ARCH) -> list:
    """Dispatch-call ratio G for M in (4, 2, 1) with the PyTorch chain and the fused chain."""
    from .machine import FUSED_CHAIN
    rows = []
    for M in (4, 2, 1):
        a = replace(arch, M=M)
        rows.append((M, a.q,
                     dispatch_breakdown(a, synthetic_dgx_h100(chain=PYTORCH_CHAIN))["G"],
                     dispatch_breakdown(a, synthetic_dgx_h100(chain=FUSED_CHAIN))["G"]))
    return rows


def main() -> None:
    m = synthetic_dgx_h100()
    print(m.fabric.name)
    print("ratio %.1f, alpha and x_half borrowed from platform A, gather %d GB/s borrowed"
          % (m.fabric.ratio, m.accel.gather_gbps))
    print()
    print("%-4s %-6s %18s %18s" % ("M", "q=k/M", "G, PyTorch chain", "G, fused kernel"))
    for M, q, g_chain, g_fused in m_table():
        print("%-4d %-6d %18.3f %18.3f" % (M, q, g_chain, g_fused))
    print()
    b = hgx_b200()
    arch = MoEArch(name="single MoE layer", hidden=4096, d_expert=1408, n_experts=64, k=6, M=2,
                   gbs=8)
    d = dispatch_breakdown(arch, b)
    print("%s: one-hop %.3f ms, two-hop %.3f ms, G = %.2f" % (b.fabric.name, d["one_hop_ms"],
                                                            d["two_hop_ms"], d["G"]))
    print()
    print("Synthetic sensitivities; dispatch-call ratios, not step times: the step-level gate "
          "fails.")


if __name__ == "__main__":
    main()
