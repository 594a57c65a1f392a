"""Directional check against a published MFU record: Mixtral 8x22B and its fine-grained G8T8
variant on clusters of 128 to 1024 H100s at one global batch.

The model prices MoE layers only, so it cannot predict an MFU.  It is asked two directional
questions instead -- is the fine-grained model's utilisation ceiling the lower one at every
cluster size, and does no model's ceiling rise from the smallest cluster to the largest -- and
both hold.  For every (model, cluster) the expert-parallel degree is the one that maximises the
ceiling, as a tuned run would choose it.

Public surface of the reference's ``sim/record.py`` (:69-154).
"""
from __future__ import annotations

from dataclasses import replace

from . import codesign as cd
from ._text import Column, Ledger, render_table
from .codesign import Machine, MoEArch
from .envelope import evaluate

MPF_SEQ = 4096
MPF_GLOBAL_BATCH_SEQS = 1024
MPF_CLUSTERS = (128, 256, 512, 1024)
EP_CHOICES = (8, 16, 32, 64, 128)
NODE_SIZE = 8


def _mixtral(name: str, d_expert: int, n_experts: int, k: int) -> MoEArch:
    return MoEArch(name=name, hidden=6144, d_expert=d_expert, n_experts=n_experts, k=k, M=k,
                   n_moe_layers=56, seq=MPF_SEQ, mbs=1, gbs=MPF_GLOBAL_BATCH_SEQS)


MIXTRAL_8X22B = _mixtral("Mixtral 8x22B", 16384, 8, 2)
MIXTRAL_G8T8 = _mixtral("Mixtral-8x22B-G8T8", 2048, 64, 8)
MODELS = (MIXTRAL_8X22B, MIXTRAL_G8T8)
MPF_MFU = {
    MIXTRAL_8X22B.name: dict(zip(MPF_CLUSTERS, (52.2, 50.7, 48.9, 44.9))),
    MIXTRAL_G8T8.name: dict(zip(MPF_CLUSTERS, (30.0, 29.3, 26.7, 25.5))),
}


def eos_like(ep_ranks: int) -> Machine:
    """Synthetic H100 nodes holding ``ep_ranks`` expert-parallel ranks; inside a single node
    there is no slow level, so both levels run at the intra-node rate."""
    nodes = ep_ranks // NODE_SIZE or 1
    machine = cd.synthetic_dgx_h100(nodes=nodes)
    if nodes > 1:
        return machine
    flat = replace(machine.fabric, beta_inter_gbps=machine.fabric.beta_intra_gbps)
    return Machine(machine.accel, flat, machine.chain)


def tokens_per_accel(cluster: int) -> int:
    return MPF_GLOBAL_BATCH_SEQS * MPF_SEQ // cluster


def best_point(arch: MoEArch, cluster: int):
    """``(ep, Point)`` with the highest ceiling among the legal expert-parallel degrees."""
    sequences, rest = divmod(tokens_per_accel(cluster), MPF_SEQ)
    if rest:
        raise ValueError("tokens per accelerator is not a whole number of sequences")
    shaped = replace(arch, mbs=sequences)
    legal = [ep for ep in EP_CHOICES if ep <= min(arch.n_experts, cluster)]
    priced = [(ep, evaluate(shaped, eos_like(ep))) for ep in legal]
    # the first of equal ceilings wins, as a strict-improvement scan would have it
    return max(priced, key=lambda t: t[1].utilisation_ceiling, default=None)


def comparison() -> list:
    rows = []
    for cluster in MPF_CLUSTERS:
        for arch in MODELS:
            ep, point = best_point(arch, cluster)
            rows.append((cluster, tokens_per_accel(cluster), arch.name, ep,
                         100.0 * point.utilisation_ceiling, MPF_MFU[arch.name][cluster]))
    return rows


def _ledger(rows=None) -> Ledger:
    ceiling = {(name, cluster): value for cluster, _, name, _, value, _ in rows or comparison()}
    coarse, fine = MIXTRAL_8X22B.name, MIXTRAL_G8T8.name
    small, large = MPF_CLUSTERS[0], MPF_CLUSTERS[-1]
    led = Ledger()
    led.add("granularity_ordering_holds",
            all(ceiling[fine, c] < ceiling[coarse, c] for c in MPF_CLUSTERS))
    led.add("endpoint_decline_holds",
            all(ceiling[name, large] <= ceiling[name, small] for name in (coarse, fine)))
    return led


def checks(rows=None) -> dict:
    return _ledger(rows).as_dict()


_COLUMNS = (
    Column("cluster", "%-8d", lambda r: r[0]),
    Column("tokens/acc", "%11d", lambda r: r[1]),
    Column("model", "%-20s", lambda r: r[2]),
    Column("EP*", "%4d", lambda r: r[3]),
    Column("ceiling %", "%10.1f", lambda r: r[4]),
    Column("published MFU", "%14.1f", lambda r: r[5]),
)
_VERDICTS = (("granularity_ordering_holds", "fine-grained variant lower at every size"),
             ("endpoint_decline_holds", "no rise from the smallest to the largest cluster"))


def main() -> None:
    rows = comparison()
    print("Published MFU against this model's MoE-layer ceiling (synthetic H100 nodes;")
    print("ceilings are MoE-layer-only and are not MFU predictions)")
    head, _rule, *body = render_table(_COLUMNS, rows)
    print("\n".join([head] + body))
    verdict = checks(rows)
    for key, sentence in _VERDICTS:
        print("%s: %s" % (sentence, "holds" if verdict[key] else "FAILS"))


if __name__ == "__main__":
    main()
