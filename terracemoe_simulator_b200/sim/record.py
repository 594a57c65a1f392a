"""Directional check against published MFU: Mixtral 8x22B against its fine-grained G8T8 variant on
128-1024 H100s.  The model prices MoE layers only, so it does not predict MFU; it is asked two
directional questions -- is the fine-grained model's ceiling lower at every cluster size, and do
the ceilings not rise from the smallest to the largest cluster -- and both hold.

Parity with the reference ``sim/record.py`` (:69-154).
"""
from __future__ import annotations

from dataclasses import replace

from .codesign import Machine, MoEArch, synthetic_dgx_h100
from .envelope import evaluate

MPF_SEQ = 4096
MPF_GLOBAL_BATCH_SEQS = 1024
MPF_CLUSTERS = (128, 256, 512, 1024)
MIXTRAL_8X22B = MoEArch(name="Mixtral 8x22B", hidden=6144, d_expert=16384, n_experts=8, k=2, M=2,
                        n_moe_layers=56, seq=MPF_SEQ, mbs=1, gbs=MPF_GLOBAL_BATCH_SEQS)
MIXTRAL_G8T8 = MoEArch(name="Mixtral-8x22B-G8T8", hidden=6144, d_expert=2048, n_experts=64, k=8,
                       M=8, n_moe_layers=56, seq=MPF_SEQ, mbs=1, gbs=MPF_GLOBAL_BATCH_SEQS)
MPF_MFU = {"Mixtral 8x22B": {128: 52.2, 256: 50.7, 512: 48.9, 1024: 44.9},
           "Mixtral-8x22B-G8T8": {128: 30.0, 256: 29.3, 512: 26.7, 1024: 25.5}}


def eos_like(ep_ranks: int) -> Machine:
    nodes = max(1, ep_ranks // 8)
    m = synthetic_dgx_h100(nodes=nodes)
    if nodes == 1:      # EP inside one node: no slow level
        m = Machine(m.accel, replace(m.fabric, beta_inter_gbps=m.fabric.beta_intra_gbps), m.chain)
    return m


def tokens_per_accel(cluster: int) -> int:
    return MPF_GLOBAL_BATCH_SEQS * MPF_SEQ // cluster


def best_point(arch: MoEArch, cluster: int):
    toks = tokens_per_accel(cluster)
    if toks % MPF_SEQ:
        raise ValueError("tokens per accelerator is not a whole number of sequences")
    a = replace(arch, mbs=toks // MPF_SEQ)
    best = None
    for ep in (8, 16, 32, 64, 128):
        if ep > arch.n_experts or ep > cluster:
            continue
        p = evaluate(a, eos_like(ep))
        if best is None or p.utilisation_ceiling > best[1].utilisation_ceiling:
            best = (ep, p)
    return best


def comparison() -> list:
    out = []
    for cluster in MPF_CLUSTERS:
        for arch in (MIXTRAL_8X22B, MIXTRAL_G8T8):
            ep, p = best_point(arch, cluster)
            out.append((cluster, tokens_per_accel(cluster), arch.name, ep,
                        100.0 * p.utilisation_ceiling, MPF_MFU[arch.name][cluster]))
    return out


def checks(rows=None) -> dict:
    by: dict = {}
    for cluster, _, name, _, ceil, _ in rows or comparison():
        by.setdefault(name, {})[cluster] = ceil
    first, last = MPF_CLUSTERS[0], MPF_CLUSTERS[-1]
    return {"granularity_ordering_holds": all(by["Mixtral-8x22B-G8T8"][c] < by["Mixtral 8x22B"][c]
                                              for c in MPF_CLUSTERS),
            "endpoint_decline_holds": all(v[last] <= v[first] for v in by.values())}


def main() -> None:
    print("Published MFU against this model's MoE-layer ceiling (synthetic H100 nodes;")
    print("ceilings are MoE-layer-only and are not MFU predictions)")
    print("%-8s %11s %-20s %4s %10s %14s" % ("cluster", "tokens/acc", "model", "EP*", "ceiling %",
                                             "published MFU"))
    for cluster, toks, name, ep, ceil, mfu in comparison():
        print("%-8d %11d %-20s %4d %10.1f %14.1f" % (cluster, toks, name, ep, ceil, mfu))
    ck = checks()
    print("fine-grained variant lower at every size: %s"
          % ("holds" if ck["granularity_ordering_holds"] else "FAILS"))
    print("no rise from the smallest to the largest cluster: %s"
          % ("holds" if ck["endpoint_decline_holds"] else "FAILS"))


if __name__ == "__main__":
    main()
