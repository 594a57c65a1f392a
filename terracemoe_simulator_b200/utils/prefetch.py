"""Host-to-device input prefetch: the copy of step i+1's batch overlaps step i's compute.

``DevicePrefetcher`` takes an iterable of pinned host tensors (or tuples of them), keeps two
device buffers, and issues every host-to-device copy on a side stream one step ahead of its use;
``next()`` makes the compute stream wait on that copy's event and immediately starts the
following copy.  On a CPU device it degenerates to passing the batches through.

The reference has no input pipeline (its only training loop builds tensors on the device,
``tests/test_checkpoint.py:16-23``); this exists so that the end-to-end numbers of the benchmarks
include the copy of every step's input without serialising it in front of the step.
"""
from __future__ import annotations

import torch


class DevicePrefetcher:
    def __init__(self, batches, device, depth: int = 2):
        self.it = iter(batches)
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.depth = max(1, depth)
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.queue = []                 # (device batch, event) in issue order
        self.copied_bytes = 0
        for _ in range(self.depth):
            self._issue()

    @staticmethod
    def _map(batch, fn):
        if isinstance(batch, (tuple, list)):
            return type(batch)(fn(t) for t in batch)
        return fn(batch)

    def _issue(self, after=None) -> None:
        try:
            host = next(self.it)
        except StopIteration:
            return
        if not self.cuda:
            self.queue.append((host, None))
            return
        if after is not None:           # start the copy only once this event has happened
            self.stream.wait_event(after)
        with torch.cuda.stream(self.stream):
            dev = self._map(host, lambda t: t.to(self.device, non_blocking=True))
            event = torch.cuda.Event()
            event.record(self.stream)
        self._map(host, lambda t: self._count(t))
        self.queue.append((dev, event))

    def _count(self, t):
        self.copied_bytes += t.numel() * t.element_size()
        return t

    def __iter__(self):
        return self

    def take(self):
        """The next batch, without starting another copy (pair with :meth:`refill`)."""
        if not self.queue:
            raise StopIteration
        dev, event = self.queue.pop(0)
        if event is not None:
            torch.cuda.current_stream(self.device).wait_event(event)
            # the buffer is consumed on the compute stream: keep the allocator from handing its
            # memory to the side stream's next copy before that work has run
            self._map(dev, lambda t: t.record_stream(torch.cuda.current_stream(self.device)) or t)
        return dev

    def refill(self, after=None) -> None:
        """Start the copy of one more batch; with ``after`` (a CUDA event) the copy engine waits
        for that point of the compute stream, which lets the caller place the transfer under a
        phase of the step that does not use the interconnect."""
        self._issue(after)

    def __next__(self):
        dev = self.take()
        self._issue()
        return dev


class DeferredScalar:
    """Device-to-host read of a per-step scalar (loss, metric) that does not stall the launch queue.

    ``push(t)`` starts a non-blocking copy of the 0-d tensor ``t`` into pinned host memory and
    returns the value pushed ``lag`` calls earlier (``None`` until then), waiting only for that
    older copy; ``flush()`` waits for the copies still in flight and returns the newest value.
    Every step's value reaches the host, ``lag`` steps late, while the host keeps launching ahead
    of the device (a lag of one bounds the run-ahead to a single step, which leaves no slack for
    host jitter when several ranks wait on one another)."""

    def __init__(self, device, dtype=torch.float32, lag: int = 1, side_stream: bool = False):
        self.cuda = torch.device(device).type == "cuda"
        # with ``side_stream`` the copy leaves the compute stream: it waits for the value on a
        # stream of its own, so the next step's first kernel does not queue behind the transfer
        self.stream = torch.cuda.Stream(device) if self.cuda and side_stream else None
        self.lag = max(1, lag)
        n = self.lag + 1
        self.slots = [torch.zeros((), dtype=dtype, pin_memory=self.cuda) for _ in range(n)]
        self.events = [None] * n
        self.n = 0
        self.bytes_per_read = self.slots[0].element_size()

    def _take(self, i):
        if self.events[i] is not None:
            self.events[i].synchronize()
        return float(self.slots[i])

    def push(self, t):
        n_slots = len(self.slots)
        i = self.n % n_slots
        prev = self._take((self.n - self.lag) % n_slots) if self.n >= self.lag else None
        value = t.detach().to(self.slots[i].dtype)
        if self.stream is not None:
            ready = torch.cuda.Event()
            ready.record()
            value.record_stream(self.stream)
            with torch.cuda.stream(self.stream):
                self.stream.wait_event(ready)
                self.slots[i].copy_(value, non_blocking=True)
                self.events[i] = torch.cuda.Event()
                self.events[i].record(self.stream)
        else:
            self.slots[i].copy_(value, non_blocking=True)
            if self.cuda:
                self.events[i] = torch.cuda.Event()
                self.events[i].record()
        self.n += 1
        return prev

    def flush(self):
        if self.n == 0:
            return None
        last = None
        for j in range(max(0, self.n - self.lag), self.n):
            last = self._take(j % len(self.slots))
        return last
