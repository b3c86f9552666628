"""Region timers (CUDA events on GPU, ``perf_counter`` on CPU) with a cross-rank report.

``timers()`` returns the process-wide registry; it is a no-op object until ``enable_timers(True)`` (the trainer's
``--timers``).  ``start(name)`` / ``stop(name)`` bracket a region on the current stream; regions nest by call order and
the report prints them as a tree with max / mean over ranks and the imbalance ``max / mean``.  This fills the role of
the AxoNN timers + Plexus ``print_axonn_timer_data`` used by the reference (``gt3d/gt3d/train/train_dist.py:598-626,
665-670``).
"""
import time
from collections import OrderedDict

import torch
import torch.distributed as dist


class _NullTimers:
    enabled = False

    def start(self, name):
        pass

    def stop(self, name):
        pass

    def reset(self):
        pass

    def region(self, name):
        return _NullRegion()


class _NullRegion:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


class _Region:
    def __init__(self, t, name):
        self.t, self.name = t, name

    def __enter__(self):
        self.t.start(self.name)
        return self

    def __exit__(self, *a):
        self.t.stop(self.name)
        return False


class RegionTimers:
    enabled = True

    def __init__(self):
        self.reset()

    def reset(self):
        self._open = {}
        self._pairs = OrderedDict()          # name -> list of (start, stop) events or float seconds
        self._depth = {}
        self._stack = []

    def _now(self):
        if torch.cuda.is_available():
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            return ev
        return time.perf_counter()

    def start(self, name):
        self._depth.setdefault(name, len(self._stack))
        self._stack.append(name)
        self._open[name] = self._now()

    def stop(self, name):
        t0 = self._open.pop(name, None)
        if t0 is None:
            return
        if self._stack and self._stack[-1] == name:
            self._stack.pop()
        elif name in self._stack:
            self._stack.remove(name)
        self._pairs.setdefault(name, []).append((t0, self._now()))

    def region(self, name):
        return _Region(self, name)

    def totals_ms(self):
        """name -> (total ms, calls); synchronises the device."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        out = OrderedDict()
        for name, pairs in self._pairs.items():
            if pairs and isinstance(pairs[0][0], float):
                tot = sum((b - a) for a, b in pairs) * 1e3
            else:
                tot = sum(a.elapsed_time(b) for a, b in pairs)
            out[name] = (tot, len(pairs))
        return out

    def report(self, divide_by=1, file=None):
        """Rank 0 prints the tree: per region max / mean over ranks (ms per ``divide_by`` steps) and the imbalance."""
        tot = self.totals_ms()
        names = list(tot.keys())
        vals = torch.tensor([tot[n][0] for n in names], dtype=torch.float64)
        world = dist.get_world_size() if dist.is_initialized() else 1
        if world > 1:
            gathered = [None] * world
            dist.all_gather_object(gathered, (names, vals.tolist()))
            if any(g[0] != names for g in gathered):
                names = [n for n in names if all(n in g[0] for g in gathered)]
            mat = torch.tensor([[dict(zip(g[0], g[1]))[n] for n in names] for g in gathered], dtype=torch.float64)
        else:
            mat = vals[None, :]
        rank = dist.get_rank() if dist.is_initialized() else 0
        lines = []
        for i, n in enumerate(names):
            mx, mean = mat[:, i].max().item() / divide_by, mat[:, i].mean().item() / divide_by
            lines.append(f"[timers] {'  ' * self._depth.get(n, 0)}{n:<44s} max {mx:9.3f} ms  mean {mean:9.3f} ms  "
                         f"imbalance {mx / mean if mean > 0 else 1.0:5.2f}  calls {tot[n][1] // max(divide_by, 1)}")
        if rank == 0:
            print("\n".join(lines), file=file, flush=True)
        return lines


_TIMERS = [_NullTimers()]


def enable_timers(on: bool = True):
    _TIMERS[0] = RegionTimers() if on else _NullTimers()
    return _TIMERS[0]


def timers():
    return _TIMERS[0]
