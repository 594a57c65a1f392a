"""Phase model skeleton: per-layer spans of the two-hop dispatch (splits read-back, Hop A,
arrival chain, Hop B, bracketed expert compute, combine) and an overlap model that REFUSES to
produce a step time until its three constants have been measured (``step_ms`` raises
``NotImplementedError`` while any is ``None``).  Keeps the failed step-level gate from being
papered over with guessed overlap numbers.

Parity with the reference ``sim/phase.py`` (:77-167).
"""
from __future__ import annotations

from dataclasses import dataclass

UNCALIBRATED = None


@dataclass
class PhaseSpans:
    splits_sync: float = 0.0
    hop_a: float = 0.0
    arrival_chain: float = 0.0
    hop_b: float = 0.0
    expert_ffn_lo: float = 0.0
    expert_ffn_hi: float = 0.0
    combine: float = 0.0

    @property
    def comm_ms(self) -> float:
        return self.splits_sync + self.hop_a + self.hop_b + self.combine

    @property
    def local_ms(self) -> float:
        return self.arrival_chain

    def compute_bracket(self):
        return self.expert_ffn_lo, self.expert_ffn_hi


@dataclass
class OverlapModel:
    overlap_efficiency: float = UNCALIBRATED
    non_moe_compute_ms: float = UNCALIBRATED
    chain_on_compute_stream: bool = UNCALIBRATED

    def missing(self) -> list:
        fields = (("overlap_efficiency", self.overlap_efficiency),
                  ("non_moe_compute_ms", self.non_moe_compute_ms),
                  ("chain_on_compute_stream", self.chain_on_compute_stream))
        return [name for name, val in fields if val is None]

    def is_calibrated(self) -> bool:
        return not self.missing()


def spans_for(cluster, geom, expert_cfg: dict) -> PhaseSpans:
    from .compute import expert_ffn
    from .core import _a2a_ms
    self_a = geom.M / geom.n_groups if geom.n_groups > 1 else 1.0
    hop_a = _a2a_ms(cluster.slow, geom.n_groups, geom.rows_hop_a(), geom.row_bytes(), self_a)
    hop_b = _a2a_ms(cluster.fast, geom.R, geom.rows_hop_b(), geom.row_bytes(), 1.0 / geom.R)
    ffn = expert_ffn(geom.tokens_per_rank, geom.k, expert_cfg["n_experts"], geom.ep, geom.H,
                     expert_cfg["d_expert"], expert_cfg.get("n_mats", 2))
    return PhaseSpans(splits_sync=cluster.splits_sync_ms, hop_a=hop_a,
                      arrival_chain=cluster.chain_us_per_row * geom.rows_hop_b() / 1000.0,
                      hop_b=hop_b, expert_ffn_lo=ffn["ms_fast"], expert_ffn_hi=ffn["ms_slow"],
                      combine=hop_a + hop_b)


def step_ms(spans: PhaseSpans, overlap: OverlapModel, microbatches: int, moe_layers: int):
    if not overlap.is_calibrated():
        raise NotImplementedError("phase model is uncalibrated; missing %s -- no step-time "
                                  "prediction until they are measured"
                                  % ", ".join(overlap.missing()))
    concurrent = overlap.non_moe_compute_ms / max(moe_layers, 1)
    if microbatches > 1:
        concurrent += spans.expert_ffn_lo * (microbatches - 1) / microbatches
    hidden = min(spans.comm_ms, concurrent * overlap.overlap_efficiency)
    local = spans.arrival_chain if overlap.chain_on_compute_stream else 0.0
    return (spans.comm_ms - hidden + local + spans.expert_ffn_lo) * moe_layers * microbatches


def report(cluster, geom, expert_cfg: dict, overlap: OverlapModel | None = None) -> dict:
    overlap = overlap or OverlapModel()
    s = spans_for(cluster, geom, expert_cfg)
    return {"spans": s, "comm_ms": s.comm_ms, "compute_bracket": s.compute_bracket(),
            "calibrated": overlap.is_calibrated(), "missing": overlap.missing()}


def main() -> None:
    from .calibrate import flat_supernode
    from .core import MoEGeometry
    g = MoEGeometry(name="n4", n_groups=4, R=8, k=6, M=2, seq=4096, mbs=1, gbs=4 * 8 * 4096)
    r = report(flat_supernode(), g, {"n_experts": 128, "d_expert": 2048})
    s = r["spans"]
    print("per-layer spans (ms): splits %.3f  hop A %.3f  chain %.3f  hop B %.3f  combine %.3f"
          % (s.splits_sync, s.hop_a, s.arrival_chain, s.hop_b, s.combine))
    print("expert FFN bracket: %.3f - %.3f ms" % s.compute_bracket())
    print("calibrated: %s; missing: %s" % (r["calibrated"], ", ".join(r["missing"])))
    print("step_ms() raises until the overlap constants are measured.")


if __name__ == "__main__":
    main()
