"""Is bandwidth across a boundary set by the bytes or by how many peers they are spread over?

Each rank sends a fixed number of bytes to the other half of the job, spread over n = 1, 2, 4 ...
peers there (explicit split sizes, rotated so that every rank also receives from exactly n
peers), and nothing to its own half.  Total bytes per rank stay fixed; only the fan-out varies.
A last phase times a plain all-to-all of the same total.  Percall style, MAX over ranks.

The reference ran this across its supernode boundary (``bench/xsupernode_peers.py:67-146``) to
show that the peer-count effect spans less than 10 %; ``sim.tiers`` records that result.  On
NVSwitch the halves are an arbitrary split of one flat domain, and the probe measures how many
concurrent peers a GPU needs to fill its 18 links.

    python -m torch.distributed.run --nproc-per-node 8 \
        -m terracemoe_simulator_b200.bench.fabric_peers --out peers.json
"""
from __future__ import annotations

import argparse
import sys

import torch
import torch.distributed as dist

from . import harness as hz

SIZES_MIB = [32, 128]
PEERS = [1, 2, 4, 8, 16, 32, 64]


def peer_splits(rank: int, world: int, n: int, chunk: int):
    """Send and receive split lists for n peers in the other half, rotation by local index."""
    half = world // 2
    local, other = rank % half, (half if rank < half else 0)
    send, recv = [0] * world, [0] * world
    for j in range(n):
        send[other + (local + j) % half] = chunk
        recv[other + (local - j) % half] = chunk
    return send, recv


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--out", required=True)
    ap.add_argument("--sizes-mib", type=float, nargs="+", default=SIZES_MIB)
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--calls", type=int, default=7)
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--tag", default="")
    args = ap.parse_args(argv)
    env = hz.init(args.cpu)
    if env.world < 2 or env.world % 2:
        raise SystemExit("needs an even number of ranks")
    half = env.world // 2
    rows = []
    for mib in args.sizes_mib:
        total = int(mib * 1024 * 1024)
        cross = total // 2
        for n in PEERS:
            if n > half or cross % (n * 32):
                continue
            chunk = cross // (n * 2)
            send, recv = peer_splits(env.rank, env.world, n, chunk)
            inp = torch.ones(n * chunk, dtype=torch.bfloat16, device=env.device)
            out = torch.empty_like(inp)
            call = lambda: dist.all_to_all_single(out, inp, recv, send)      # noqa: E731
            for _ in range(3):
                call()
            ms, sp = hz.median_of(env, hz.percall, call, args.calls, args.repeats)
            rows.append({"phase": "peers", "peers": n, "bytes": total, "cross_bytes": cross,
                         "ms": ms, "spread": sp, "gbs": cross / (ms * 1e-3) / 1e9})
            hz.say(env, "  %6.1f MiB  %3d peer(s) across  %8.4f ms  %7.1f GB/s per rank (spread %4.1f%%)"
                   % (mib, n, ms, rows[-1]["gbs"], 100 * sp))
            del inp, out
        if (total // 2) % env.world == 0:
            gi = torch.ones(total // 2, dtype=torch.bfloat16, device=env.device)
            go = torch.empty_like(gi)
            gcall = lambda: dist.all_to_all_single(go, gi)                   # noqa: E731
            for _ in range(3):
                gcall()
            ms, sp = hz.median_of(env, hz.percall, gcall, args.calls, args.repeats)
            rows.append({"phase": "global", "peers": env.world - 1, "bytes": total,
                         "cross_bytes": total // 2, "ms": ms, "spread": sp})
            hz.say(env, "  %6.1f MiB  plain all-to-all over %d ranks  %8.4f ms" % (mib, env.world, ms))
            del gi, go
    peer_ms = [r["ms"] for r in rows if r["phase"] == "peers" and r["bytes"] == rows[0]["bytes"]]
    span = max(peer_ms) / min(peer_ms) if peer_ms else 1.0
    hz.say(env, "peer-count effect at the smallest size: %.2fx between best and worst fan-out" % span)
    hz.write_json(env, args.out, {"tag": args.tag, "world": env.world, "rows": rows,
                                  "peer_effect_span": span})
    hz.finish(env)
    return 0


if __name__ == "__main__":
    sys.exit(main())
