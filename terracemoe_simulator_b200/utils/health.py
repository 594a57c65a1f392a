"""Host-side failure detection for ranks that spin on each other's flags.

The fused expert-parallel kernels wait (bounded) for flags that peer GPUs raise.  A peer that has
left turns every such wait into a timeout a couple of seconds long, so the ranks should learn of
it on the host, *between* steps and before their next launch.  ``Heartbeat`` does that over any
``torch.distributed`` store (the ``TCPStore`` of the process group's rendezvous, a ``FileStore``,
a ``HashStore`` in tests):

    hb = Heartbeat(store, rank, world, interval_s=0.5)      # starts a daemon thread that beats
    ...
    hb.guard()            # before a step: raises PeerLost naming the ranks that left or went quiet
    ...
    hb.leave()            # a rank that stops between steps says so; peers see it at once

A beat is a counter per rank that only grows (``store.add``); a rank is *quiet* when its counter
has not moved for ``timeout_s`` by this rank's clock, and *gone* when it announced its leave.  No
device call is made anywhere in this module, and nothing here faults or hangs a GPU: a detected
loss is an exception on the host, after which the caller tears the arena down
(``FusedEPContext.rebuild``) or restarts from a checkpoint.

The reference has no failure detection (its observed hangs were spin-waits,
``docs/08-onesided.md:60-82``); this is the host half of the bounded-wait design.
"""
from __future__ import annotations

import threading
import time


class PeerLost(RuntimeError):
    def __init__(self, gone, quiet):
        self.gone, self.quiet = sorted(gone), sorted(quiet)
        parts = []
        if self.gone:
            parts.append("left: %s" % self.gone)
        if self.quiet:
            parts.append("no heartbeat: %s" % self.quiet)
        super().__init__("expert-parallel peers lost (%s)" % "; ".join(parts))


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 0.5,
                 timeout_s: float = 5.0, prefix: str = "terrace/hb", start: bool = True,
                 clock=time.monotonic):
        if timeout_s <= interval_s:
            raise ValueError("timeout_s must exceed interval_s")
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s, self.prefix, self.clock = interval_s, timeout_s, prefix, clock
        self._stop = threading.Event()
        self._thread = None
        self._seen = {}            # rank -> (last counter value, local time it changed)
        self._left = False
        self.beat()                # every key exists before anybody reads it
        if start:
            self._thread = threading.Thread(target=self._run, name="terrace-heartbeat", daemon=True)
            self._thread.start()

    # ---- this rank ---------------------------------------------------------------------------
    def _key(self, rank: int, what: str = "beat") -> str:
        return "%s/%s/%d" % (self.prefix, what, rank)

    def beat(self) -> int:
        return int(self.store.add(self._key(self.rank), 1))

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                self.beat()
            except Exception:          # noqa: BLE001  (the store went away: stop quietly)
                return

    def leave(self) -> None:
        """Announce that this rank stops taking part (call between steps, with none of this
        rank's kernels or collectives in flight)."""
        self._left = True
        self.store.add(self._key(self.rank, "left"), 1)
        self.stop()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None and self._thread is not threading.current_thread():
            self._thread.join(timeout=2 * self.interval_s + 1.0)

    # ---- the peers ---------------------------------------------------------------------------
    def _counter(self, rank: int, what: str) -> int:
        return int(self.store.add(self._key(rank, what), 0))       # add 0 = read, creates at 0

    def check(self):
        """``(gone, quiet)``: ranks that announced their leave, and ranks whose counter has not
        moved for ``timeout_s``.  A rank never seen beating counts from the first check."""
        now = self.clock()
        gone, quiet = [], []
        for r in range(self.world):
            if r == self.rank:
                continue
            if self._counter(r, "left") > 0:
                gone.append(r)
                continue
            value = self._counter(r, "beat")
            last = self._seen.get(r)
            if last is None or value != last[0]:
                self._seen[r] = (value, now)
            elif now - last[1] > self.timeout_s:
                quiet.append(r)
        return gone, quiet

    def guard(self) -> None:
        """Raise ``PeerLost`` if any peer left or went quiet; call before every step's launches."""
        if self._left:
            raise RuntimeError("this rank has left the group")
        gone, quiet = self.check()
        if gone or quiet:
            raise PeerLost(gone, quiet)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.stop()
        return False
