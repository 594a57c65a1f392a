"""NVLink roofline of the fused dispatch + combine on 8 x B200: bytes that must leave a GPU,
the time they need at the measured peer-copy rate, and what the measured calls achieve.

    python -m terracemoe_simulator_b200.sim.b200_roofline

Byte ledger per GPU and direction (uniform routing, bf16 rows of ``H`` elements):

    one-hop   T * k rows, of which 1 - 1 / world leave the GPU
    two-hop   Hop A: T * M rows, of which 1 - 1 / N_g leave (the own group's representative is
              local only when it is the GPU itself, i.e. the share is counted per group)
              Hop B: T * k rows forwarded by the representative, of which 1 - 1 / R leave; with
              GPU-level dedup one copy per (row, owner GPU): T * M * D(q) rows instead of T * k

A dispatch + combine call moves the ledger twice (there and back).  The roofline time is the
ledger over the measured peer-copy bandwidth of 770 GB/s per direction (nominal 900); the
achieved fraction is roofline time over measured time.  For a two-hop call the two hops use the
same egress port one after the other, so their bytes add.

The reference has no such ledger in code; its byte criterion is the closed form of
``tools/breakeven.py`` (:61-79), with which this module is cross-checked by the tests.
"""
from __future__ import annotations

from .calibrate import load_b200_sweep

PEER_COPY_GBPS = 770.0          # measured peer copy, per direction per GPU
NOMINAL_GBPS = 900.0
BYTES_PER_ELEM = 2


def distinct_gpus(q: int, R: int, epr: int) -> float:
    """Expected number of distinct GPUs of a group that q distinct experts of it sit on."""
    from ..tools.breakeven import D_of
    return D_of(q, R, epr)


def egress_bytes(path: str, tokens: int, k: int, M: int, hidden: int, world: int, R: int,
                 dedup: bool = False, epr: int = 8) -> dict:
    """Bytes leaving one GPU in one direction (dispatch OR combine)."""
    row = hidden * BYTES_PER_ELEM
    if path == "one_hop":
        out = tokens * k * (1.0 - 1.0 / world) * row
        return {"hop_a": 0.0, "hop_b": 0.0, "total": out}
    if path != "two_hop":
        raise ValueError("path must be one_hop or two_hop")
    n_groups = world // R
    q = k // M
    hop_a = tokens * M * (1.0 - 1.0 / n_groups) * row
    per_row = distinct_gpus(q, R, epr) if dedup else q
    hop_b = tokens * M * per_row * (1.0 - 1.0 / R) * row
    return {"hop_a": hop_a, "hop_b": hop_b, "total": hop_a + hop_b}


def roofline_ms(nbytes: float, gbps: float = PEER_COPY_GBPS) -> float:
    return nbytes / (gbps * 1e6)


def table(rows=None) -> list:
    """One line per sweep point: ledger, roofline time of a dispatch + combine call, measured
    time, achieved fraction, for the fused one-hop and two-hop calls and the NCCL arm."""
    out = []
    for r in (load_b200_sweep() if rows is None else rows):
        args = (r["tokens"], r["k"], r["M"], r["hidden"], r["world"], r["R"])
        one = egress_bytes("one_hop", *args)["total"]
        two = egress_bytes("two_hop", *args)["total"]
        t1, t2 = 2.0 * roofline_ms(one), 2.0 * roofline_ms(two)
        out.append({"R": r["R"], "q": r["q"], "tokens": r["tokens"],
                    "one_hop_mb": one / 1e6, "two_hop_mb": two / 1e6,
                    "one_hop_frac": t1 / r["one_hop_ms"], "two_hop_frac": t2 / r["two_hop_ms"],
                    "nccl_frac": t1 / r["nccl_a2a_x2_ms"],
                    "one_hop_ms": r["one_hop_ms"], "two_hop_ms": r["two_hop_ms"]})
    return out


def main() -> None:
    print("fused dispatch + combine on 8 x B200: achieved fraction of the NVLink roofline")
    print("(bytes leaving a GPU, there and back, over %.0f GB/s measured per direction)"
          % PEER_COPY_GBPS)
    print("%2s %2s %6s %9s %9s %9s %9s %9s" % ("R", "q", "tok", "1hop MB", "2hop MB", "1hop frac",
                                              "2hop frac", "NCCL frac"))
    for t in table():
        if t["tokens"] < 4096:
            continue
        print("%2d %2d %6d %9.1f %9.1f %9.2f %9.2f %9.2f"
              % (t["R"], t["q"], t["tokens"], t["one_hop_mb"], t["two_hop_mb"], t["one_hop_frac"],
                 t["two_hop_frac"], t["nccl_frac"]))
    big = [t for t in table() if t["tokens"] == 16384]
    print("at 16384 tokens per GPU: one-hop %.2f-%.2f of the roofline, NCCL %.2f-%.2f"
          % (min(t["one_hop_frac"] for t in big), max(t["one_hop_frac"] for t in big),
             min(t["nccl_frac"] for t in big), max(t["nccl_frac"] for t in big)))
    print("two-hop with groups of one GPU moves 1 / q of the bytes; its fraction is low because")
    print("the q-fold expansion inside the representative runs at HBM speed, not on the links.")


if __name__ == "__main__":
    main()
