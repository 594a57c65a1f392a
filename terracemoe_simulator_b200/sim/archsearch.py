"""Architecture search at fixed capacity: the granularity family (E x g, d_expert / g, k x g keeps
total and active parameters) crossed with every group cap M that divides k.  Candidates are
ranked by dispatch + expert time with nothing overlapped -- an upper bound, not a step time.
Quality is not priced.

Parity with the reference ``sim/archsearch.py`` (``Candidate`` :46-63, ``granularity_family``
:70-87, ``evaluate`` :90-115, ``search`` / ``rank`` / ``table`` :118-165).
"""
from __future__ import annotations

from dataclasses import dataclass, replace

from .codesign import (UNMEASURED, Machine, MemoryProfile, MoEArch, dispatch_breakdown,
                       expert_matmul, min_ep_for_memory)


@dataclass(frozen=True)
class Candidate:
    arch: MoEArch
    granularity: float
    one_hop_ms: float
    two_hop_ms: float
    best_dispatch_ms: float
    strategy: str
    expert_ms: float
    expert_bound_by: str
    min_ep: int
    feasible: bool
    reason: str = ""

    @property
    def no_overlap_ms(self) -> float:
        return self.best_dispatch_ms + self.expert_ms


def _divisors(n: int):
    return [d for d in range(1, n + 1) if n % d == 0]


def granularity_family(base: MoEArch, factors=(0.5, 1, 2, 4, 8)):
    cap_total, cap_active = base.n_experts * base.d_expert, base.k * base.d_expert
    out = []
    for g in factors:
        E, d, k = (int(round(base.n_experts * g)), int(round(base.d_expert / g)),
                   int(round(base.k * g)))
        if min(E, d, k) < 1 or k > E:
            continue
        if abs(E * d - cap_total) > 0.01 * cap_total or abs(k * d - cap_active) > 0.01 * cap_active:
            continue
        out.append((g, replace(base, name="%s-g%g" % (base.name, g), n_experts=E, d_expert=d,
                               k=k)))
    return out


def evaluate(arch: MoEArch, machine: Machine, mem: MemoryProfile = UNMEASURED) -> Candidate:
    floor = min_ep_for_memory(arch, machine, mem)["min_ep"]
    feasible = 0 < floor <= machine.fabric.ep
    reason = "" if feasible else "experts need EP %d, fabric has %d" % (floor, machine.fabric.ep)
    mm = expert_matmul(arch, machine, machine.fabric.ep)
    d = dispatch_breakdown(arch, machine)
    applies = d["domain_condition"] and d["fanout_condition"]
    if applies and d["two_hop_ms"] < d["one_hop_ms"]:
        best, strategy = d["two_hop_ms"], "two-hop"
    else:
        best, strategy = d["one_hop_ms"], "one-hop"
        if not applies:
            why = "expert parallelism fits one fast domain" if not d["domain_condition"] else \
                "q = k/M is 1, nothing to deduplicate"
            reason = (reason + "; " if reason else "") + "two-hop does not apply: " + why
    return Candidate(arch=arch, granularity=0.0, one_hop_ms=d["one_hop_ms"],
                     two_hop_ms=d["two_hop_ms"], best_dispatch_ms=best, strategy=strategy,
                     expert_ms=mm["ms"], expert_bound_by=mm["bound_by"], min_ep=floor,
                     feasible=feasible, reason=reason)


def search(base: MoEArch, machine: Machine, granularities=(0.5, 1, 2, 4, 8), hiddens=None,
           mem: MemoryProfile = UNMEASURED) -> list:
    out = []
    for g, arch in granularity_family(base, granularities):
        for M in _divisors(arch.k):
            if M <= machine.fabric.nodes:
                cand = evaluate(replace(arch, name="%s-M%d" % (arch.name, M), M=M), machine, mem)
                out.append(replace(cand, granularity=g))
    for H in hiddens or ():
        for M in _divisors(base.k):
            if M <= machine.fabric.nodes:
                cand = evaluate(replace(base, name="%s-H%d-M%d" % (base.name, H, M), hidden=H,
                                        M=M), machine, mem)
                out.append(replace(cand, granularity=1.0))
    return out


def rank(cands, key="no_overlap_ms", feasible_only: bool = True) -> list:
    pool = [c for c in cands if c.feasible] if feasible_only else list(cands)
    return sorted(pool, key=lambda c: getattr(c, key))


def table(cands, top: int = 12) -> str:
    lines = ["%-6s %-7s %-7s %-4s %-4s %-4s %10s %10s %10s %-9s"
             % ("gran", "experts", "d_exp", "k", "M", "q", "dispatch", "expert", "sum(UB)",
                "strategy"), "-" * 88]
    for c in rank(cands)[:top]:
        a = c.arch
        lines.append("%-6g %-7d %-7d %-4d %-4d %-4d %10.3f %10.3f %10.3f %-9s"
                     % (c.granularity, a.n_experts, a.d_expert, a.k, a.M, a.q, c.best_dispatch_ms,
                        c.expert_ms, c.no_overlap_ms, c.strategy))
    lines += ["", "sum(UB) is dispatch plus expert with nothing overlapped, an upper bound and "
                  "not a step time: the step-level gate fails."]
    return "\n".join(lines)


def main() -> None:
    from .codesign import REFERENCE_ARCH, synthetic_dgx_h100
    m = synthetic_dgx_h100()
    print("Granularity x group-cap search at the reference capacity on the %s" % m.fabric.name)
    print("(synthetic sensitivity; quality of each point is NOT priced)")
    print()
    print(table(search(REFERENCE_ARCH, m)))


if __name__ == "__main__":
    main()
