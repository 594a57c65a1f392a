"""Architecture search at fixed capacity, priced on one machine.

The search space is a lattice: the granularity axis (experts x g, expert width / g, top-k x g:
total and active parameters stay put), crossed with every group cap M that divides k and fits
the fabric's group count, plus an optional hidden-width axis (which moves capacity and is to be
read separately).  Each lattice point becomes a ``Candidate`` carrying its dispatch time (the
better of one-hop and two-hop, when two-hop applies at all), its expert time and the smallest
expert-parallel degree its weights fit in.  The sort key is dispatch + expert with nothing
overlapped: an upper bound that is loose in the same direction everywhere, not a step time.
Quality is not priced.

Public surface of the reference's ``sim/archsearch.py`` (``Candidate`` :46-63,
``granularity_family`` :70-87, ``evaluate`` :90-115, ``search`` / ``rank`` / ``table``
:118-165).
"""
from __future__ import annotations

import itertools
import operator
from dataclasses import dataclass, replace

from . import codesign as cd
from ._text import Column, render_table
from .codesign import UNMEASURED, Machine, MemoryProfile, MoEArch

DEFAULT_FACTORS = (0.5, 1, 2, 4, 8)
CAPACITY_TOLERANCE = 0.01       # rounding may move either capacity product by at most 1 %


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
    small = [d for d in range(1, int(n ** 0.5) + 1) if n % d == 0]
    return sorted(set(small) | {n // d for d in small})


def _scaled(base: MoEArch, g: float):
    """``base`` moved by granularity ``g``, or None when the point is illegal or rounding broke
    one of the two capacity invariants."""
    shape = {"n_experts": round(base.n_experts * g), "d_expert": round(base.d_expert / g),
             "k": round(base.k * g)}
    if min(shape.values()) < 1 or shape["k"] > shape["n_experts"]:
        return None
    for width_of in ("n_experts", "k"):               # total, then active parameters
        kept, want = shape[width_of] * shape["d_expert"], getattr(base, width_of) * base.d_expert
        if abs(kept - want) > CAPACITY_TOLERANCE * want:
            return None
    return replace(base, name="%s-g%g" % (base.name, g), **{k: int(v) for k, v in shape.items()})


def granularity_family(base: MoEArch, factors=DEFAULT_FACTORS):
    scaled = ((g, _scaled(base, g)) for g in factors)
    return [(g, arch) for g, arch in scaled if arch is not None]


def _why_not_two_hop(d: dict) -> str:
    if not d["domain_condition"]:
        return "two-hop does not apply: expert parallelism fits one fast domain"
    return "two-hop does not apply: q = k/M is 1, nothing to deduplicate"


def evaluate(arch: MoEArch, machine: Machine, mem: MemoryProfile = UNMEASURED) -> Candidate:
    ep = machine.fabric.ep
    need = cd.min_ep_for_memory(arch, machine, mem)["min_ep"]
    experts = cd.expert_matmul(arch, machine, ep)
    hops = cd.dispatch_breakdown(arch, machine)
    notes = []
    fits = 0 < need <= ep
    if not fits:
        notes.append("experts need EP %d, fabric has %d" % (need, ep))
    eligible = hops["domain_condition"] and hops["fanout_condition"]
    use_two = eligible and hops["two_hop_ms"] < hops["one_hop_ms"]
    if not eligible:
        notes.append(_why_not_two_hop(hops))
    chosen = "two_hop_ms" if use_two else "one_hop_ms"
    priced = {name: hops[name] for name in ("one_hop_ms", "two_hop_ms")}
    priced.update(best_dispatch_ms=hops[chosen], strategy=chosen[:3] + "-hop",
                  expert_ms=experts["ms"], expert_bound_by=experts["bound_by"])
    return Candidate(arch, 0.0, min_ep=need, feasible=fits, reason="; ".join(notes), **priced)


def _lattice(base: MoEArch, machine: Machine, granularities, hiddens):
    """``(granularity, architecture)`` for every point of the search lattice."""
    groups = machine.fabric.nodes
    for g, arch in granularity_family(base, granularities):
        for M in _divisors(arch.k):
            if M <= groups:
                yield g, replace(arch, name="%s-M%d" % (arch.name, M), M=M)
    for H, M in itertools.product(hiddens or (), _divisors(base.k)):
        if M <= groups:
            yield 1.0, replace(base, name="%s-H%d-M%d" % (base.name, H, M), hidden=H, M=M)


def search(base: MoEArch, machine: Machine, granularities=DEFAULT_FACTORS, hiddens=None,
           mem: MemoryProfile = UNMEASURED) -> list:
    return [replace(evaluate(arch, machine, mem), granularity=g)
            for g, arch in _lattice(base, machine, granularities, hiddens)]


def rank(cands, key="no_overlap_ms", feasible_only: bool = True) -> list:
    keep = filter(operator.attrgetter("feasible"), cands) if feasible_only else cands
    return sorted(keep, key=operator.attrgetter(key))


_COLUMNS = (
    Column("gran", "%-6g", lambda c: c.granularity),
    Column("experts", "%-7d", lambda c: c.arch.n_experts),
    Column("d_exp", "%-7d", lambda c: c.arch.d_expert),
    Column("k", "%-4d", lambda c: c.arch.k),
    Column("M", "%-4d", lambda c: c.arch.M),
    Column("q", "%-4d", lambda c: c.arch.q),
    Column("dispatch", "%10.3f", lambda c: c.best_dispatch_ms),
    Column("expert", "%10.3f", lambda c: c.expert_ms),
    Column("sum(UB)", "%10.3f", lambda c: c.no_overlap_ms),
    Column("strategy", "%-9s", lambda c: c.strategy),
)
_FOOTNOTE = ("sum(UB) is dispatch plus expert with nothing overlapped, an upper bound and not a "
             "step time: the step-level gate fails.")


def table(cands, top: int = 12) -> str:
    return "\n".join(render_table(_COLUMNS, rank(cands)[:top], rule=88) + ["", _FOOTNOTE])


def main() -> None:
    m = cd.synthetic_dgx_h100()
    print("Granularity x group-cap search at the reference capacity on the %s" % m.fabric.name)
    print("(synthetic sensitivity; quality of each point is NOT priced)")
    print()
    print(table(search(cd.REFERENCE_ARCH, m)))
    b = cd.hgx_b200()
    print()
    print("Same search on the %s (measured fabric: one NVSwitch domain, logical groups)"
          % b.fabric.name)
    print()
    print(table(search(cd.REFERENCE_ARCH, b)))


if __name__ == "__main__":
    main()
