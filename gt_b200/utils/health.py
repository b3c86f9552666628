"""Host-side failure detection for long multi-rank runs.

The kernels of this package never wait for a peer without a limit: a device-side wait that expires writes a code into the
per-device status word and the kernel returns (``gt_b200.ops.native.check_status`` turns it into an exception after the
next synchronisation).  This module adds the host half, so that a rank that has died, hung or left is noticed BEFORE the
next step launches collectives that would need it:

* ``Heartbeat``: every rank bumps a counter in the job's key-value store once per step; ``check()`` raises
  ``PeerFailure`` naming the ranks that announced a failure or whose counter has not moved for ``timeout`` seconds.
* ``leave()`` / ``fail(reason)``: a rank announces that it is going away (between steps, nothing in flight).
* ``guarded(fn)``: run a step; on any exception announce the failure to the peers, then re-raise.

The reference has no failure handling (a failed rank kills the job by the launcher's timeout, ``gt3d/scripts/
run_dac26_strategies.sh:22,31``).  Everything here is host code over ``torch.distributed``'s store; it launches nothing.
"""
import time

import torch.distributed as dist


class PeerFailure(RuntimeError):
    def __init__(self, ranks, why):
        super().__init__(f"ranks {sorted(ranks)} are not alive: {why}")
        self.ranks = sorted(ranks)


class Heartbeat:
    def __init__(self, store=None, rank=None, world=None, timeout=30.0, prefix="gt_hb"):
        self.store = store if store is not None else dist.distributed_c10d._get_default_store()
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.timeout, self.prefix = float(timeout), prefix
        self.count = 0
        self._seen = {r: (-1, time.monotonic()) for r in range(self.world)}
        self.store.set(self._key(self.rank), "0")

    def _key(self, r, what="beat"):
        return f"{self.prefix}/{what}/{r}"

    def beat(self):
        """Call once per step (host side, before the step's launches)."""
        self.count += 1
        self.store.set(self._key(self.rank), str(self.count))

    def fail(self, reason="failed"):
        self.store.set(self._key(self.rank, "gone"), str(reason))

    def leave(self):
        self.fail("left")

    def check(self, wait_for_first=0.0):
        """Raise ``PeerFailure`` if a peer announced its departure or has been silent for ``timeout`` seconds."""
        now = time.monotonic()
        gone, silent = {}, {}
        for r in range(self.world):
            if r == self.rank:
                continue
            if self.store.num_keys() and self._has(self._key(r, "gone")):
                gone[r] = self.store.get(self._key(r, "gone")).decode()
                continue
            cur = int(self.store.get(self._key(r)).decode()) if self._has(self._key(r)) else -1
            last, t_last = self._seen[r]
            if cur != last:
                self._seen[r] = (cur, now)
            elif now - t_last > self.timeout + wait_for_first:
                silent[r] = now - t_last
        if gone:
            raise PeerFailure(gone, "; ".join(f"rank {r}: {why}" for r, why in sorted(gone.items())))
        if silent:
            raise PeerFailure(silent, "; ".join(f"rank {r} silent for {s:.1f} s" for r, s in sorted(silent.items())))

    def _has(self, key):
        try:
            return bool(self.store.check([key]))
        except Exception:
            return False

    def guarded(self, fn, *a, **kw):
        try:
            return fn(*a, **kw)
        except BaseException as exc:                      # announce, then propagate
            try:
                self.fail(f"{type(exc).__name__}: {exc}"[:200])
            finally:
                raise
