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
        previous = reader.push(loss)          # float of the previous step's loss (None the first time)
    last = reader.flush()

On a CPU device both classes degrade to plain synchronous behaviour.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch


class DevicePrefetcher:
    """Copies tuples of pinned host tensors to the device on a side stream.  4-D floating-point
    tensors can be converted to channels-last on that stream as well."""

    def __init__(self, device: torch.device, channels_last: bool = True):
        self.device = torch.device(device)
        self.channels_last = channels_last
        self._cuda = self.device.type == "cuda"
        self._stream = torch.cuda.Stream(self.device) if self._cuda else None
        self._next: Optional[Tuple[Sequence[torch.Tensor], Optional[torch.cuda.Event]]] = None

    def put(self, *host_tensors: torch.Tensor) -> None:
        if not self._cuda:
            self._next = (tuple(host_tensors), None)
            return
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
    pushed one step earlier (whose copy has long finished)."""

    def __init__(self, device: torch.device):
        self.device = torch.device(device)
        self._cuda = self.device.type == "cuda"
        self._slots = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)] if self._cuda else None
        self._events = [None, None]
        self._i = 0
        self._pending: Optional[int] = None
        self._cpu_value: Optional[float] = None

    def _take(self) -> Optional[float]:
        if not self._cuda:
            v, self._cpu_value = self._cpu_value, None
            return v
        if self._pending is None:
            return None
        k = self._pending
        self._pending = None
        self._events[k].synchronize()
        return float(self._slots[k][0])

    def push(self, scalar: torch.Tensor) -> Optional[float]:
        previous = self._take()
        if not self._cuda:
            self._cpu_value = float(scalar.detach())
            return previous
        k = self._i
        self._i ^= 1
        self._slots[k].copy_(scalar.detach().reshape(1).float(), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self._events[k] = ev
        self._pending = k
        return previous

    def flush(self) -> Optional[float]:
        """Value of the last push (waits for it)."""
        return self._take()
