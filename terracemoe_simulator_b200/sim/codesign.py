"""Co-design layer: one MoE architecture on one machine (accelerator + fabric + arrival chain).

For an (architecture, machine) pair it answers, term by term, what binds first: whether the
expert weights are resident at all (``residency`` / ``min_ep_for_memory``), what the expert
matmuls of one rank and layer cost and whether compute or memory bounds them
(``expert_matmul``), and what one dispatch costs one-hop and two-hop (``dispatch_breakdown``).
The terms are per call and per layer and are deliberately NOT added into a step time: the
step-level gate of the model fails.

The descriptions themselves (``MoEArch``, ``Fabric``, ``Machine``, ``MemoryProfile``) are plain
dataclasses kept in ``sim/archtypes.py`` and re-exported here.
``synthetic_dgx_h100`` is a datasheet machine for sensitivity studies; ``hgx_b200`` is the box
this repository measures on (one NVSwitch domain, logical groups, fused arrival chain).

Public surface of the reference's ``sim/codesign.py``: ``MoEArch`` / ``Fabric`` / ``Machine``
:56-173, ``expert_matmul`` :180-222, ``MemoryProfile`` / ``UNMEASURED`` / ``residency`` /
``min_ep_for_memory`` :229-317, ``dispatch_breakdown`` :324-361, ``profile`` / ``sweep``
:364-401, ``synthetic_dgx_h100`` :408-438, ``REFERENCE_ARCH`` / ``m_table`` :442-460.
"""
from __future__ import annotations

from dataclasses import replace

from . import compute
from .archtypes import UNMEASURED, Fabric, Machine, MemoryProfile, MoEArch  # noqa: F401
from .compute import INDEX_RULE, INDEX_RULE_ERROR, PEAK_TFLOPS
from .core import ClusterSpec, MoEGeometry, one_hop_call, two_hop_call
from .machine import PYTORCH_CHAIN, Accelerator, ArrivalChain

GIB = float(1 << 30)
MEASURED_ROWS_FLOOR = 1536        # smallest rows-per-expert the GEMM table was measured at


def expert_matmul(arch: MoEArch, machine: Machine, ep: int, backward: bool = False) -> dict:
    """Routed experts of one rank and one layer: the slower of a compute-bound time (measured
    GEMM efficiency curve, rescaled to the machine's peak) and a memory-bound time (weights plus
    activations once through HBM)."""
    local, rows = compute._local_shape(arch.tokens_per_rank, arch.k, arch.n_experts, ep)
    passes = 1.0 + bool(backward)
    elem = arch.bytes_per_elem
    flops = 2.0 * rows * arch.hidden * arch.d_expert * arch.n_mats * local * passes
    rate = compute.efficiency_bracket(rows, arch.hidden, arch.d_expert)["per_rule"][INDEX_RULE]
    rate *= machine.peak_tflops / PEAK_TFLOPS
    moved = (local * arch.params_per_expert() * elem * passes                 # weights
             + rows * local * (arch.hidden + 2.0 * arch.d_expert) * elem)    # activations
    t = {"compute": compute._ms(flops, rate), "memory": moved / (machine.accel.hbm_gbps * 1e6)}
    binding = max(("compute", "memory"), key=t.get)      # a tie reads "compute"
    return {
        "rows_per_expert": rows, "experts_local": local, "flops": flops,
        "ms_compute_bound": t["compute"], "ms_memory_bound": t["memory"], "ms": t[binding],
        "bound_by": binding, "arithmetic_intensity": rows,
        "machine_balance": machine.balance_flops_per_byte,
        "compute_measured": rows >= MEASURED_ROWS_FLOOR and not machine.transfers_compute,
        "roofline_borrowed": not machine.transfers_compute, "tflops_rule": INDEX_RULE,
        "tflops_worst_error": INDEX_RULE_ERROR["worst"],
    }


def residency(arch: MoEArch, machine: Machine, ep: int, profile: MemoryProfile = UNMEASURED,
              non_expert_params: int = 0) -> dict:
    """Bytes one accelerator must hold at expert-parallel degree ``ep``, component by component,
    each with the provenance of its number."""
    capacity = machine.accel.hbm_capacity_gb * 1e9
    per_param = arch.bytes_per_elem + arch.optimizer_bytes_per_param
    held = {
        "expert_bytes": arch.expert_bytes_all_layers(with_optimizer=True) / ep,
        "non_expert_bytes": non_expert_params * per_param,
        "activation_bytes": (profile.activation_bytes_per_token_layer * arch.tokens_per_rank
                             * arch.n_moe_layers),
        "overhead_bytes": capacity * profile.overhead_frac,
    }
    total = sum(held.values())
    where = {
        "expert_bytes": "computed from the architecture and the optimizer",
        "non_expert_bytes": "computed" if non_expert_params
        else "NOT SUPPLIED: attention and embeddings omitted",
        "activation_bytes": profile.provenance(), "overhead_bytes": profile.provenance(),
    }
    return dict(held, total_bytes=total, capacity_bytes=capacity, fits=total <= capacity,
                headroom_bytes=capacity - total, provenance=where, measured=profile.measured,
                profile=profile.name)


def min_ep_for_memory(arch: MoEArch, machine: Machine, profile: MemoryProfile = UNMEASURED,
                      non_expert_params: int = 0) -> dict:
    """Smallest power-of-two expert-parallel degree (or, failing those, one expert per rank) at
    which the residency fits; -1 when not even that does."""
    degrees, ep = [], 1
    while ep < arch.n_experts:
        degrees.append(ep)
        ep *= 2
    degrees.append(arch.n_experts)
    for ep in degrees:
        res = residency(arch, machine, ep, profile, non_expert_params)
        if res["fits"]:
            break
    else:
        ep = -1
    return {"min_ep": ep, "residency": res, "measured": res["measured"]}


def _cluster(arch: MoEArch, machine: Machine, chain_us_per_row: float) -> ClusterSpec:
    f = machine.fabric
    return ClusterSpec(name=f.name, R=f.cards_per_node, chain_us_per_row=chain_us_per_row,
                       **f.levels())


def _geometry(arch: MoEArch, fabric: Fabric) -> MoEGeometry:
    return MoEGeometry(name=arch.name, n_groups=fabric.nodes, R=fabric.cards_per_node, k=arch.k,
                       M=arch.M, H=arch.hidden, seq=arch.seq, mbs=arch.mbs, gbs=arch.gbs,
                       moe_layers=arch.n_moe_layers, bytes_per_elem=arch.bytes_per_elem)


def dispatch_breakdown(arch: MoEArch, machine: Machine) -> dict:
    """One dispatch call both ways, with the arrival chain priced by the machine's chain tier,
    and the two structural conditions under which two-hop is an option at all."""
    fabric = machine.fabric
    pairs = arch.tokens_per_rank * arch.k
    chain_ms = machine.chain.ms(pairs, arch.hidden, machine.accel)
    per_row_us = 1e3 * chain_ms / pairs
    cluster, geom = _cluster(arch, machine, per_row_us), _geometry(arch, fabric)
    one, two = one_hop_call(cluster, geom), two_hop_call(cluster, geom)
    return {"ep": fabric.ep, "q": arch.q, "ratio": fabric.ratio, "one_hop_ms": one,
            "two_hop_ms": two, "G": one / two, "chain_us_per_row": per_row_us,
            "chain_ms": chain_ms, "chain_share_of_two_hop": chain_ms / two,
            "domain_condition": fabric.ep > fabric.cards_per_node,
            "fanout_condition": arch.q >= 2}


_BINDS = {"memory": "expert matmul, memory bound", "compute": "expert matmul, compute bound"}


def profile(arch: MoEArch, machine: Machine, mem: MemoryProfile = UNMEASURED,
            non_expert_params: int = 0) -> dict:
    ep = machine.fabric.ep
    need = min_ep_for_memory(arch, machine, mem, non_expert_params)
    fits = 0 < need["min_ep"] <= ep
    matmul = expert_matmul(arch, machine, ep)
    warning = None if need["measured"] else (
        "the residency verdict rests on an unmeasured memory profile (docs/11-residency.md lists "
        "what has to be measured)")
    return {
        "arch": arch.name, "machine": machine.fabric.name,
        "memory": {"min_ep": need["min_ep"], "configured_ep": ep, "fits": fits,
                   "measured": need["measured"], "breakdown": need["residency"],
                   "expert_gib": arch.expert_bytes_all_layers() / GIB},
        "expert_matmul": matmul, "dispatch": dispatch_breakdown(arch, machine),
        "binds": _BINDS[matmul["bound_by"]] if fits else "memory capacity",
        "caveat": "step-level composition is behind a failing gate; the terms above are per-call "
                  "and per-layer and do not add to a step time",
        "memory_caveat": warning,
    }


def sweep(base: MoEArch, machine: Machine, knob: str, values, mem: MemoryProfile = UNMEASURED):
    """``[(value, profile or {"error": ...})]`` for one field of the architecture."""
    def one(value):
        try:
            return profile(replace(base, **{knob: value}), machine, mem)
        except ValueError as exc:
            return {"error": str(exc)}
    return [(v, one(v)) for v in values]


def synthetic_dgx_h100(nodes: int = 16, chain: ArrivalChain = PYTORCH_CHAIN) -> Machine:
    """Datasheet H100 nodes behind NDR400; gather and launch constants borrowed from platform A."""
    from . import calibrate as cal
    from .machine import GATHER_GBPS_MEASURED
    h100 = Accelerator.from_gather_bw(
        "synthetic H100 SXM", gather_gbps=GATHER_GBPS_MEASURED, hbm_capacity_gb=80.0,
        launch_ms=0.129, hbm_gbps=3350.0, peak_tflops=989.0,
        notes="vendor datasheet numbers; gather and launch borrowed from platform A")
    ndr = Fabric("synthetic DGX H100 + NDR400, %d nodes" % nodes, 8, nodes, beta_intra_gbps=450.0,
                 beta_inter_gbps=50.0, alpha_ms=tuple(cal.ALPHA_PTS),
                 x_half_bytes=float(cal.X_HALF_FLAT))
    return Machine(h100, ndr, chain)


def hgx_b200(group_size: int = 2, chain: ArrivalChain | None = None) -> Machine:
    """One 8 x B200 box: a single NVSwitch domain split into logical groups of ``group_size``.
    Both "levels" run at the same measured rate and one fixed cost applies at every world."""
    from . import calibrate as cal
    from .machine import B200, B200_FUSED
    groups = 8 // group_size
    fixed_ms = cal.B200_ALPHA_US["flat"] * 1e-3
    switch = Fabric("HGX B200, %d logical groups of %d" % (groups, group_size), group_size, groups,
                    beta_intra_gbps=cal.B200_BETA_GBPS, beta_inter_gbps=cal.B200_BETA_GBPS,
                    alpha_ms=((2, fixed_ms), (16, fixed_ms)),
                    x_half_bytes=float(cal.B200_X_HALF))
    return Machine(B200, switch, chain if chain is not None else B200_FUSED)


REFERENCE_ARCH = MoEArch(name="reference", hidden=7168, d_expert=2048, n_experts=256, k=8, M=4,
                         n_moe_layers=1, seq=4096, mbs=1)
BENCH_LAYER = MoEArch(name="single MoE layer", hidden=4096, d_expert=1408, n_experts=64, k=6, M=2,
                      gbs=8)


def b200_layer(arch: MoEArch = BENCH_LAYER, group_size: int = 2, chunks: int = 2) -> dict:
    """Forward pass of one MoE layer on the 8 x B200 box under this repository's overlap
    schedule: measured grouped-GEMM throughput for the experts, the calibrated fabric for the
    dispatch, and ``phase.ChunkedSchedule`` for what of the communication stays exposed.  Unlike
    the platform-A terms above these DO add up, because the overlap is fixed by the launch order
    rather than fitted; ``sim/b200_step.py`` checks the sum against measured steps."""
    from .phase import ChunkedSchedule
    machine = hgx_b200(group_size)
    ep = machine.fabric.ep
    experts = compute.expert_ffn_b200(arch.tokens_per_rank, arch.k, arch.n_experts, ep,
                                      arch.hidden, arch.d_expert)
    hops = dispatch_breakdown(arch, machine)
    schedule = ChunkedSchedule(chunks=chunks)
    layers = {}
    for name in ("one_hop", "two_hop"):
        there = hops[name + "_ms"]
        layers[name] = {"dispatch_ms": there, "serial_ms": experts["ms"] + 2.0 * there,
                        "exposed_ms": schedule.exposed_ms(there, experts["ms"], there),
                        "layer_ms": schedule.layer_ms(there, experts["ms"], there)}
    return {"machine": machine.fabric.name, "expert_ms": experts["ms"],
            "expert_tflops": experts["tflops"], "chunks": chunks, **layers}


def m_table(arch: MoEArch = REFERENCE_ARCH) -> list:
    """Dispatch-call ratio G for M in (4, 2, 1) with the PyTorch chain and the fused chain."""
    from .machine import FUSED_CHAIN
    machines = [synthetic_dgx_h100(chain=tier) for tier in (PYTORCH_CHAIN, FUSED_CHAIN)]
    rows = []
    for M in (4, 2, 1):
        shaped = replace(arch, M=M)
        rows.append((M, shaped.q) + tuple(dispatch_breakdown(shaped, m)["G"] for m in machines))
    return rows


def main() -> None:
    h100, b200 = synthetic_dgx_h100(), hgx_b200()
    out = [h100.fabric.name,
           "ratio %.1f, alpha and x_half borrowed from platform A, gather %d GB/s borrowed"
           % (h100.fabric.ratio, h100.accel.gather_gbps), "",
           "%-4s %-6s %18s %18s" % ("M", "q=k/M", "G, PyTorch chain", "G, fused kernel")]
    out += ["%-4d %-6d %18.3f %18.3f" % row for row in m_table()]
    d = dispatch_breakdown(BENCH_LAYER, b200)
    out += ["", "%s: one-hop %.3f ms, two-hop %.3f ms, G = %.2f"
            % (b200.fabric.name, d["one_hop_ms"], d["two_hop_ms"], d["G"])]
    est = b200_layer()
    out += ["  forward layer, %d push chunks: experts %.3f ms; one-hop %.3f ms (%.3f exposed, "
            "%.3f if nothing overlapped); two-hop %.3f ms"
            % (est["chunks"], est["expert_ms"], est["one_hop"]["layer_ms"],
               est["one_hop"]["exposed_ms"], est["one_hop"]["serial_ms"],
               est["two_hop"]["layer_ms"]), "",
            "Synthetic sensitivities; dispatch-call ratios, not step times: the step-level gate "
            "fails."]
    print("\n".join(out))


if __name__ == "__main__":
    main()
