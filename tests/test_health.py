"""Host-side failure detection: heartbeats over a torch.distributed store (no GPU involved)."""
import os
import tempfile
import time

import pytest
import torch.distributed as dist

from terracemoe_simulator_b200.utils.health import Heartbeat, PeerLost


class _Clock:
    def __init__(self):
        self.t = 0.0

    def __call__(self):
        return self.t


def test_quiet_peer_is_detected_after_the_timeout_and_not_before():
    store, clock = dist.HashStore(), _Clock()
    hbs = [Heartbeat(store, r, 3, interval_s=0.1, timeout_s=1.0, start=False, clock=clock)
           for r in range(3)]
    hbs[0].guard()                                   # first look: everybody counts from now
    clock.t = 0.9
    hbs[1].beat()                                    # rank 1 keeps beating, rank 2 does not
    hbs[0].guard()
    clock.t = 1.5
    hbs[1].beat()
    with pytest.raises(PeerLost) as err:
        hbs[0].guard()
    assert err.value.quiet == [2] and err.value.gone == []
    hbs[2].beat()                                    # it comes back: no longer quiet
    assert hbs[0].check() == ([], [])


def test_announced_leave_is_seen_at_once_and_the_leaver_cannot_guard():
    store = dist.HashStore()
    a = Heartbeat(store, 0, 2, start=False)
    b = Heartbeat(store, 1, 2, start=False)
    a.guard()
    b.leave()
    with pytest.raises(PeerLost) as err:
        a.guard()
    assert err.value.gone == [1] and "left" in str(err.value)
    with pytest.raises(RuntimeError):
        b.guard()
    with pytest.raises(ValueError):
        Heartbeat(store, 0, 2, interval_s=1.0, timeout_s=0.5, start=False)


def test_background_thread_beats_and_stops():
    store = dist.HashStore()
    with Heartbeat(store, 0, 2, interval_s=0.02, timeout_s=0.3) as a:
        watcher = Heartbeat(store, 1, 2, interval_s=0.02, timeout_s=0.3, start=False)
        watcher.check()
        time.sleep(0.15)
        first = watcher._counter(0, "beat")
        assert first >= 2                            # the daemon thread has been beating
        assert watcher.check() == ([], [])
    time.sleep(0.1)
    assert watcher._counter(0, "beat") <= first + 1  # stopped with the context
    watcher.check()                                  # takes note of a last beat, if there was one
    time.sleep(0.4)
    assert watcher.check() == ([], [0])              # and is reported quiet after the timeout


def _proc(rank, world, path, queue):
    store = dist.FileStore(path, world)
    hb = Heartbeat(store, rank, world, interval_s=0.05, timeout_s=30.0)
    try:
        if rank == 1:                                # leaves once both peers have stepped
            deadline = time.monotonic() + 60
            while int(store.add("ready", 0)) < world - 1 and time.monotonic() < deadline:
                time.sleep(0.02)
            hb.leave()
            queue.put((rank, "left"))
            return
        for step in range(2000):
            try:
                hb.guard()
            except PeerLost as exc:
                queue.put((rank, "lost", exc.gone, exc.quiet, step))
                return
            if step == 0:
                store.add("ready", 1)                # one clean step done
            time.sleep(0.02)
        queue.put((rank, "never noticed"))
    finally:
        hb.stop()


def test_processes_learn_of_a_leaving_rank_before_their_next_step():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "store")
        procs = [ctx.Process(target=_proc, args=(r, 3, path, q)) for r in range(3)]
        for p in procs:
            p.start()
        out = sorted(q.get(timeout=120) for _ in range(3))
        for p in procs:
            p.join(timeout=30)
    assert out[1] == (1, "left")
    for r in (0, 2):
        assert out[r][:3] == (r, "lost", [1]) and out[r][4] > 0, out


def _trace_proc(rank, world, port, queue):
    import os as _os
    import torch.distributed as _dist
    _os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), TERRACE_TRACE="events")
    _dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from terracemoe_simulator_b200.utils import trace
        trace.reset()
        with trace.phase("work", cuda=False):
            time.sleep(0.05 * (rank + 1))                # rank 1 is the slow one
        rep = trace.report(group=True)
        queue.put((rank, rep["work"]["ms"], rep["work"]["calls"]))
    finally:
        _dist.destroy_process_group()


def test_trace_report_is_the_max_over_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_trace_proc, args=(r, 2, 29433, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    assert out[0][1] == out[1][1] >= 95.0                # both report the slow rank's 100 ms
    assert out[0][2] == out[1][2] == 1
