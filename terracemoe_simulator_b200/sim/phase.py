"""Phase model skeleton: the spans of one MoE layer under two-hop dispatch, and an overlap model
that refuses to turn them into a step time before it has been measured.

The spans (per layer, ms): splits read-back, Hop A, arrival chain, Hop B, the routed experts
(bracketed between the fastest and slowest reading of the GEMM curve) and the combine, which
retraces both hops.  ``OverlapModel`` holds the three constants a step time would need -- how
efficiently communication hides behind concurrent compute, how much non-MoE compute a layer
offers for hiding, and whether the arrival chain occupies the compute stream -- and
``step_ms`` raises ``NotImplementedError`` while any of them is unset.  That keeps the failed
step-level gate from being papered over with guessed overlap numbers.  (On the B200 transport
of this repository the overlap is a property of the schedule and is measured directly; see
``sim/b200_step.py``.)

Public surface of the reference's ``sim/phase.py`` (:77-167).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass

UNCALIBRATED = None


SPAN_NAMES = ("splits_sync", "hop_a", "arrival_chain", "hop_b", "expert_ffn_lo", "expert_ffn_hi",
              "combine")
_ON_THE_WIRE = ("splits_sync", "hop_a", "hop_b", "combine")


def _comm_ms(self) -> float:
    return sum(getattr(self, name) for name in _ON_THE_WIRE)


# one float per span, all defaulting to zero (ms per layer and micro-batch, nothing overlapped)
PhaseSpans = dataclasses.make_dataclass(
    "PhaseSpans", [(name, float, 0.0) for name in SPAN_NAMES],
    namespace={"comm_ms": property(_comm_ms),
               "local_ms": property(lambda self: self.arrival_chain),
               "compute_bracket": lambda self: (self.expert_ffn_lo, self.expert_ffn_hi)})


@dataclass
class OverlapModel:
    overlap_efficiency: float = UNCALIBRATED
    non_moe_compute_ms: float = UNCALIBRATED
    chain_on_compute_stream: bool = UNCALIBRATED

    def missing(self) -> list:
        return [f.name for f in dataclasses.fields(self) if getattr(self, f.name) is UNCALIBRATED]

    def is_calibrated(self) -> bool:
        return not self.missing()

    def require(self) -> None:
        gaps = self.missing()
        if gaps:
            raise NotImplementedError("phase model is uncalibrated; missing %s -- no step-time "
                                      "prediction until they are measured" % ", ".join(gaps))


def spans_for(cluster, geom, expert_cfg: dict) -> PhaseSpans:
    from .compute import expert_ffn
    from .imbalance import exchanges
    hops = exchanges(cluster, geom)
    row = geom.row_bytes()
    there = {name: hops[name].ms(row) for name in ("hop_a", "hop_b")}
    ffn = expert_ffn(geom.tokens_per_rank, geom.k, expert_cfg["n_experts"], geom.ep, geom.H,
                     expert_cfg["d_expert"], expert_cfg.get("n_mats", 2))
    return PhaseSpans(splits_sync=cluster.splits_sync_ms,
                      arrival_chain=cluster.chain_us_per_row * geom.rows_hop_b() * 1e-3,
                      expert_ffn_lo=ffn["ms_fast"], expert_ffn_hi=ffn["ms_slow"],
                      combine=sum(there.values()), **there)


def step_ms(spans: PhaseSpans, overlap: OverlapModel, microbatches: int, moe_layers: int):
    """Step time of the MoE layers once the overlap constants are known: per layer and
    micro-batch, the communication that does not hide, the chain when it blocks the compute
    stream, and the (fast reading of the) expert compute."""
    overlap.require()
    layers = moe_layers if moe_layers > 1 else 1
    cover = overlap.non_moe_compute_ms / layers
    if microbatches > 1:       # another micro-batch's experts run meanwhile
        cover += spans.expert_ffn_lo * (1.0 - 1.0 / microbatches)
    exposed = spans.comm_ms - min(spans.comm_ms, overlap.overlap_efficiency * cover)
    blocking = spans.arrival_chain * bool(overlap.chain_on_compute_stream)
    return (exposed + blocking + spans.expert_ffn_lo) * moe_layers * microbatches


@dataclass(frozen=True)
class ChunkedSchedule:
    """The schedule of this repository's fused transport, where the overlap is not a fitted
    efficiency but a consequence of the launch order: the dispatch goes out in ``chunks`` pushes
    on a side stream and the GEMMs of chunk c run while chunk c + 1 travels; the return leg is
    written by the second GEMM's epilogue.  Exposed per direction: the first chunk's share of the
    dispatch, whatever a later chunk's transfer exceeds the GEMM time it hides under, the part
    of the return transfer the epilogue does not hide, and the final local reduction.

    ``return_hidden`` is measured, not derived: the scattering epilogue stores 8 KiB rows over
    NVLink from the same warps that drain the accumulators, so the second GEMM stretches while
    it sends; on B200 about a third of the return transfer disappears under it (2- and 4-GPU steps,
    ``sim/b200_step.py``)."""
    chunks: int = 2
    local_reduce_ms: float = 0.05
    return_hidden: float = 0.3

    def exposed_ms(self, dispatch_ms: float, expert_ms: float, return_ms: float = 0.0) -> float:
        n = max(int(self.chunks), 1)
        per_chunk_push, per_chunk_gemm = dispatch_ms / n, expert_ms / n
        spill = max(per_chunk_push - per_chunk_gemm, 0.0) * (n - 1)
        # the return transfer rides in GEMM 2's epilogue (a third of the expert time at most)
        tail = max(return_ms * (1.0 - self.return_hidden), return_ms - expert_ms / 3.0, 0.0)
        return per_chunk_push + spill + tail + self.local_reduce_ms

    def layer_ms(self, dispatch_ms: float, expert_ms: float, return_ms: float = 0.0) -> float:
        return expert_ms + self.exposed_ms(dispatch_ms, expert_ms, return_ms)


def report(cluster, geom, expert_cfg: dict, overlap: OverlapModel | None = None) -> dict:
    model = overlap if overlap is not None else OverlapModel()
    spans = spans_for(cluster, geom, expert_cfg)
    return {"spans": spans, "comm_ms": spans.comm_ms, "compute_bracket": spans.compute_bracket(),
            "calibrated": model.is_calibrated(), "missing": model.missing()}


def main() -> None:
    from .calibrate import flat_supernode
    from .core import MoEGeometry
    geom = MoEGeometry(name="n4", n_groups=4, R=8, k=6, M=2, seq=4096, mbs=1, gbs=4 * 8 * 4096)
    r = report(flat_supernode(), geom, {"n_experts": 128, "d_expert": 2048})
    shown = ("splits_sync", "hop_a", "arrival_chain", "hop_b", "combine")
    print("per-layer spans (ms): splits %.3f  hop A %.3f  chain %.3f  hop B %.3f  combine %.3f"
          % tuple(getattr(r["spans"], name) for name in shown))
    print("expert FFN bracket: %.3f - %.3f ms" % r["compute_bracket"])
    print("calibrated: %s; missing: %s" % (r["calibrated"], ", ".join(r["missing"])))
    print("step_ms() raises until the overlap constants are measured.")


if __name__ == "__main__":
    main()
