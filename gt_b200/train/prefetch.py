"""Host -> device input pipeline and pipelined result reads for a step that runs from a CUDA graph.

A captured step reads its inputs at fixed device addresses.  :class:`InputPrefetcher` keeps those static tensors and, next to
them, one staging copy on the device: the pinned host tensors of step ``i + 1`` are copied to the staging buffers on a copy
stream while step ``i`` computes; ``next()`` then waits for that copy on the compute stream and moves staging -> static
tensors device-to-device (tens of microseconds for tens of MB) before the step is launched, so the PCIe transfer is off the
critical path although every step gets freshly copied inputs.

:class:`AsyncScalar` is the matching device -> host side: the step's loss is copied into pinned memory behind the step and read
one step later, so the host never blocks on the step it has just launched.

    pre = InputPrefetcher({"x": x_host, "y": y_host}, device)   # pinned host tensors
    res = AsyncScalar(device)
    for _ in range(steps):
        inputs = pre.next(following=None)                       # static device tensors, refreshed; ``following``: other pinned
                                                                # tensors to transfer for the step after this one
        res.push(engine.train_step(loss_fn))
        value = res.pop_previous()                              # loss of the previous step (None at the first step)
    last = res.drain()

On CPU tensors both classes degrade to plain copies.
"""
import torch


class InputPrefetcher:
    def __init__(self, host_tensors, device):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.host = dict(host_tensors)
        self.static = {k: torch.empty_like(t, device=self.device) for k, t in self.host.items()}
        if self.cuda:
            for k, t in self.host.items():
                if not t.is_pinned():
                    raise ValueError(f"input '{k}' must live in pinned host memory")
            self.staging = {k: torch.empty_like(t, device=self.device) for k, t in self.host.items()}
            self.stream = torch.cuda.Stream(device=self.device)
            self.ready = torch.cuda.Event()
            self.consumed = torch.cuda.Event()
            self.consumed.record(torch.cuda.current_stream(self.device))
            self._in_flight = False
        self.bytes_per_step = sum(t.numel() * t.element_size() for t in self.host.values())

    def stage(self, host_tensors=None):
        """Start copying the inputs of the NEXT step to the device (pinned host -> staging, on the copy stream)."""
        if host_tensors is not None:
            self.host.update(host_tensors)
        if not self.cuda:
            return
        self.stream.wait_event(self.consumed)              # the previous staging contents have been moved out
        with torch.cuda.stream(self.stream):
            for k, t in self.host.items():
                self.staging[k].copy_(t, non_blocking=True)
            self.ready.record(self.stream)
        self._in_flight = True

    def next(self, following=None):
        """Static device tensors holding the inputs staged last (stages them now if nothing is in flight).  Before returning, the
        transfer for the step after this one is started: from ``following`` (a dict of pinned host tensors) if given, else from
        the same host tensors again."""
        if not self.cuda:
            for k, t in self.host.items():
                self.static[k].copy_(t)
            if following is not None:
                self.host.update(following)
            return self.static
        if not self._in_flight:
            self.stage()
        cur = torch.cuda.current_stream(self.device)
        cur.wait_event(self.ready)
        for k in self.static:
            self.static[k].copy_(self.staging[k], non_blocking=True)
        self.consumed.record(cur)
        self._in_flight = False
        self.stage(following)                               # overlap the next transfer with the step about to be launched
        return self.static


class AsyncScalar:
    """Ring of pinned host slots for per-step scalars: ``push`` copies a device scalar behind the work that produced it,
    ``pop_previous`` returns the value pushed one call earlier (waiting only for that older copy)."""

    def __init__(self, device, slots=4):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.buf = torch.zeros(slots, dtype=torch.float32)
        if self.cuda:
            self.buf = self.buf.pin_memory()
        self.events = [torch.cuda.Event() if self.cuda else None for _ in range(slots)]
        self.head = 0                                       # number of pushes
        self.read = 0                                       # number of values handed out
        self.bytes_per_step = 4

    def push(self, scalar):
        i = self.head % self.buf.numel()
        if self.head - self.read >= self.buf.numel():
            raise RuntimeError("AsyncScalar ring is full: pop before pushing more")
        self.buf[i:i + 1].copy_(scalar.detach().reshape(1).float(), non_blocking=True)
        if self.cuda:
            self.events[i].record(torch.cuda.current_stream(self.device))
        self.head += 1

    def _get(self):
        i = self.read % self.buf.numel()
        if self.cuda:
            self.events[i].synchronize()
        self.read += 1
        return float(self.buf[i])

    def pop_previous(self):
        """Value pushed before the latest one, or ``None`` if there is none yet."""
        return self._get() if self.head - self.read >= 2 else None

    def drain(self):
        """All values not handed out yet, oldest first."""
        out = []
        while self.read < self.head:
            out.append(self._get())
        return out
