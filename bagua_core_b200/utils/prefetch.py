"""Input and result pipelining for a training loop: copy the next batch from pinned host memory
while the current step computes, and read a step's loss one step late, so that neither the
host→device copy nor the device→host read ever stalls the GPU or the launching thread.

    pf = DevicePrefetcher(device)
    reader = LaggedScalarReader(device)
    pf.put(host_x, host_y)
    for ...:
        x, y = pf.get()
        pf.put(next_host_x, next_host_y)      # overlaps the step below
        loss = train_step(x, y)
        previous = reader.push(loss)          # float of an earlier step's loss (None at first)
    last = reader.flush()

On a CPU device both classes degrade to plain synchronous behaviour.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch


class DevicePrefetcher:
    """Copies tuples of pinned host tensors to the device on a side stream.  4-D floating-point
    tensors can be converted to channels-last on that stream as well."""

    def __init__(self, device: torch.device, channels_last: bool = True, after_current_work: bool = True):
        """after_current_work: the copy starts only when the work queued so far on the calling stream has
        finished.  Called at the top of a step, that places the copy of the next batch under this step's
        forward pass, when no gradient traffic is in flight, instead of wherever the launching thread's
        lead over the GPU happens to put it (the copy engines that move the batch also move the gradient
        buckets of the copy-engine all-reduce, and an unordered copy can land in front of them)."""
        self.device = torch.device(device)
        self.channels_last = channels_last
        self.after_current_work = after_current_work
        self._cuda = self.device.type == "cuda"
        self._stream = torch.cuda.Stream(self.device) if self._cuda else None
        self._next: Optional[Tuple[Sequence[torch.Tensor], Optional[torch.cuda.Event]]] = None

    def put(self, *host_tensors: torch.Tensor) -> None:
        if not self._cuda:
            self._next = (tuple(host_tensors), None)
            return
        if self.after_current_work:
            self._stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self._stream):
            out = []
            for h in host_tensors:
                d = h.to(self.device, non_blocking=True)
                if self.channels_last and d.dim() == 4 and d.is_floating_point():
                    d = d.contiguous(memory_format=torch.channels_last)
                out.append(d)
            ev = torch.cuda.Event()
            ev.record(self._stream)
        self._next = (tuple(out), ev)

    def get(self) -> Tuple[torch.Tensor, ...]:
        if self._next is None:
            raise RuntimeError("DevicePrefetcher.get() without a preceding put()")
        tensors, ev = self._next
        self._next = None
        if ev is not None:
            cur = torch.cuda.current_stream(self.device)
            cur.wait_event(ev)
            for t in tensors:
                t.record_stream(cur)  # allocated on the side stream, consumed on this one
        return tuple(tensors)


class LaggedScalarReader:
    """Reads one device scalar per step without waiting for the step that produced it: `push`
    starts an asynchronous copy of this step's scalar into pinned memory and returns the value
    pushed `lag` steps earlier (whose copy has long finished), so the launching thread may run up
    to `lag` steps ahead of the GPU and a hiccup of the host does not idle the device.  `flush`
    returns the values still outstanding; every pushed scalar is read exactly once."""

    def __init__(self, device: torch.device, lag: int = 1):
        self.device = torch.device(device)
        self.lag = max(1, int(lag))
        self._cuda = self.device.type == "cuda"
        n = self.lag + 1
        self._slots = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(n)] if self._cuda else None
        self._events = [None] * n
        self._i = 0
        self._pending = []  # slot indices (or CPU values) in push order

    def _take(self) -> Optional[float]:
        if not self._pending:
            return None
        k = self._pending.pop(0)
        if not self._cuda:
            return k
        self._events[k].synchronize()
        return float(self._slots[k][0])

    def push(self, scalar: torch.Tensor) -> Optional[float]:
        previous = self._take() if len(self._pending) >= self.lag else None
        if not self._cuda:
            self._pending.append(float(scalar.detach()))
            return previous
        k = self._i
        self._i = (self._i + 1) % len(self._slots)
        self._slots[k].copy_(scalar.detach().reshape(1).float(), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self._events[k] = ev
        self._pending.append(k)
        return previous

    def flush(self) -> Optional[float]:
        """Reads every outstanding value (waits for them); returns the last one."""
        last = None
        while self._pending:
            last = self._take()
        return last
