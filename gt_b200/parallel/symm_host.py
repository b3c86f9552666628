"""Host emulation of the symmetric heap: the peer-memory transport of :mod:`gt_b200.parallel.symm` between CPU processes.

``HostSymmetricHeap`` is the :class:`~gt_b200.parallel.symm.SymmetricHeap` with its device parts replaced: every rank's heap is
a file mapped ``MAP_SHARED`` (under ``/dev/shm`` when present) that the other ranks of the machine map too, an "address" is
``(owner rank + 1) << 44 | offset``, and the handful of native entry points the heap calls (``heap_*``, ``tensor_from_ptr``,
``group_barrier``, the ``pull_*`` kernels, the channel kernels and the two-shot all-reduce) are restated in a few lines of
torch each (:class:`HostExt`).  Everything above that line is the production code, unchanged: the bump allocator and its
allocation log, staging copies and their alternation, the barriers' placement, peer tables, the sparse plans' pull state, the
routing in ``parallel/collectives.py`` and ``parallel/sparse_comm.py``.  The ranks are real processes that run concurrently, the
flags are real words in shared memory, and every wait is bounded and records ``100 + peer`` in the status word when it expires.

What it is for: the multi-rank logic of the transport can be tested where there are fewer GPUs than ranks, or none
(``tests/test_host_heap.py``: every collective against gloo on 2 x 2 grids with unequal row groups, the allocation logs of all
ranks compared, the distributed model parity cases in double precision with the heap transport switched on, and the fused 2D
layer as one operator, whose kernels :mod:`gt_b200.parallel.fused_host` restates in torch, on grids up to 4 x 2).  What it does
not cover: the device kernels themselves (their index arithmetic, their memory ordering on a GPU), which the GPU tests cover.

The reference's pull collectives have no host mode (``gt3d/gt3d/dist/pullcomm/__init__.py:40-80`` needs NVSHMEM and GPUs).
"""
import atexit
import os
import tempfile
import time

import torch
import torch.distributed as dist

from ..ops import native
from .fused_host import FusedKernelsHost
from .symm import SymmetricHeap

_SHIFT = 44
_MASK = (1 << _SHIFT) - 1
_TYPES = {0: torch.float32, 1: torch.bfloat16, 2: torch.int32, 3: torch.int64, 4: torch.uint8, 5: torch.float64}


def _unlink(path):
    try:
        os.unlink(path)
    except OSError:
        pass


class HostExt(FusedKernelsHost):
    """The entry points of the native module that the symmetric heap uses, on shared host memory (plus, from the mixin, the
    kernels of the fused layer restated in torch)."""

    def __init__(self, rank, wait_seconds=20.0):
        self.rank, self.wait_seconds = int(rank), float(wait_seconds)
        self.segments = {}                                   # base address -> uint8 tensor over the mapped file
        self.paths = {}
        self._mod = self                                     # native.check_status looks for optional entry points here
        self.log = None                                      # a list: record every access to heap memory and every signal / wait

    # ---- recording (tests compare the recorded sequence with the protocol model) -----------------------------------------------------
    def _note(self, *event):
        if self.log is not None:
            self.log.append(event)

    def _place(self, where):
        """``(owner rank, offset)`` of an address or of a tensor that lives in a mapped heap; ``None`` for other tensors."""
        if isinstance(where, torch.Tensor) and where.numel() != 1:
            a = where.data_ptr()
            for base, seg in self.segments.items():
                if seg.data_ptr() <= a < seg.data_ptr() + seg.numel():
                    return (base >> _SHIFT) - 1, a - seg.data_ptr()
            return None
        ptr = int(where)
        return (ptr >> _SHIFT) - 1, ptr & _MASK

    def _access(self, kind, where, nbytes=None):
        """Record ``(kind, owner rank, offset, bytes)`` for an address or a tensor inside a heap."""
        if self.log is not None:
            at = self._place(where)
            if at is not None:
                if nbytes is None:
                    nbytes = where.numel() * where.element_size()
                self.log.append((kind,) + at + (int(nbytes),))

    # ---- heap management ---------------------------------------------------------------------------------------------------
    def heap_alloc(self, nbytes):
        root = "/dev/shm" if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else tempfile.gettempdir()
        fd, path = tempfile.mkstemp(prefix=f"gt_b200_heap_r{self.rank}_", dir=root)
        os.ftruncate(fd, int(nbytes))                        # zero-filled
        os.close(fd)
        base = (self.rank + 1) << _SHIFT
        self.segments[base] = torch.from_file(path, shared=True, size=int(nbytes), dtype=torch.uint8)
        self.paths[base] = path
        atexit.register(_unlink, path)                       # a rank that ends with an exception never reaches heap_free
        return base

    def heap_ipc_handle(self, base):
        return f"{self.rank}:{self.segments[base].numel()}:{self.paths[base]}".encode()

    def heap_open(self, handle):
        rank, nbytes, path = handle.decode().split(":", 2)
        base = (int(rank) + 1) << _SHIFT
        self.segments[base] = torch.from_file(path, shared=True, size=int(nbytes), dtype=torch.uint8)
        return base

    def heap_close(self, base):
        self.segments.pop(base, None)

    def heap_free(self, base):
        self.segments.pop(base, None)
        path = self.paths.pop(base, None)
        if path:
            _unlink(path)

    def _typed(self, ptr, numel, dtype, kind=None):
        """Typed view of ``numel`` elements at an address; ``kind`` ('read' / 'write') records the access."""
        ptr = int(ptr)
        seg = self.segments[ptr >> _SHIFT << _SHIFT]
        off = ptr & _MASK
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        if kind is not None:
            self._access(kind, ptr, nbytes)
        if off + nbytes > seg.numel():
            raise IndexError(f"access of {nbytes} bytes at offset {off} leaves the heap of rank {(ptr >> _SHIFT) - 1}")
        return seg[off:off + nbytes].view(dtype)

    def tensor_from_ptr(self, ptr, shape, dtype_code, device_index):
        n = 1
        for s in shape:
            n *= int(s)
        return self._typed(ptr, n, _TYPES[int(dtype_code)], "view").view(*shape)

    # ---- ordering ----------------------------------------------------------------------------------------------------------
    def _wait(self, flags, n_peers, epoch, status, note=True):
        deadline = time.monotonic() + self.wait_seconds
        for p in range(n_peers):
            if note and self.log is not None:
                self._note("wait", self._place(flags)[1], p)
            while int(flags[p]) < epoch:
                if time.monotonic() > deadline:
                    status.fill_(100 + p)
                    return
                time.sleep(0)

    def group_barrier(self, peer_flag_ptrs, my_flags, counter, me, max_spins, status):
        epoch = int(counter) + 1
        counter.fill_(epoch)
        n = peer_flag_ptrs.numel()
        for p in range(n):
            self._typed(peer_flag_ptrs[p], 64, torch.int32)[me] = epoch
        if self.log is not None:
            self._note("barrier", self._place(my_flags)[1], tuple((int(q) >> _SHIFT) - 1 for q in peer_flag_ptrs))
        self._wait(my_flags, n, epoch, status, note=False)

    def channel_signal(self, ptrs, me, counter):
        epoch = int(counter) + 1
        counter.fill_(epoch)
        self._note("signal", int(ptrs[0]) & _MASK, tuple((int(q) >> _SHIFT) - 1 for q in ptrs))
        for p in ptrs:
            self._typed(p, 8, torch.int32)[me] = epoch

    def channel_wait(self, flags, counter, n_peers, max_spins, status):
        self._wait(flags, n_peers, int(counter), status)

    # ---- collectives as reads of the owners' memory (fp32 accumulation in a fixed peer order; fp64 stays fp64) --------------------
    @staticmethod
    def _acc_type(dtype):
        return torch.float64 if dtype == torch.float64 else torch.float32

    def pull_all_gather(self, table, out):
        n = table.numel()
        chunk = out.numel() // n
        flat = out.view(n, chunk)
        for p in range(n):
            flat[p] = self._typed(table[p], chunk, out.dtype, "read")

    def pull_reduce_scatter(self, table, me, out):
        n, chunk = table.numel(), out.numel()
        acc = torch.zeros(chunk, dtype=self._acc_type(out.dtype))
        for p in range(n):
            acc += self._typed(table[p], n * chunk, out.dtype, "read")[me * chunk:(me + 1) * chunk].to(acc.dtype)
        out.view(-1).copy_(acc)

    def pull_all_reduce(self, table, out):
        acc = torch.zeros(out.numel(), dtype=self._acc_type(out.dtype))
        for p in range(table.numel()):
            acc += self._typed(table[p], out.numel(), out.dtype, "read").to(acc.dtype)
        out.view(-1).copy_(acc)

    def pull_all_to_all(self, table, me, rows, slab_bytes, to_heads, out):
        n = table.numel()
        slab = int(slab_bytes) // out.element_size()
        for p in range(n):
            src = self._typed(table[p], rows * n * slab, out.dtype, "read")
            if to_heads:                                     # rows of peer p, my head slab
                out.view(n, rows, slab)[p] = src.view(rows, n, slab)[:, me]
            else:                                            # my rows, peer p's head slab
                out.view(rows, n, slab)[:, p] = src.view(n, rows, slab)[me]

    def pull_gather_rows(self, table, owner, row, out):
        width = out.shape[1]
        for p in range(table.numel()):
            sel = torch.nonzero(owner == p).squeeze(1)
            if sel.numel():
                rows = row[sel].long()
                src = self._typed(table[p], (int(rows.max()) + 1) * width, out.dtype, "read").view(-1, width)
                out[sel] = src[rows]

    def pull_reduce_rows(self, table, src, out):
        width = out.shape[1]
        acc = torch.zeros(out.shape, dtype=self._acc_type(out.dtype))
        for p in range(table.numel()):
            idx = src[p].long()
            sel = torch.nonzero(idx >= 0).squeeze(1)
            if sel.numel():
                rows = idx[sel]
                buf = self._typed(table[p], (int(rows.max()) + 1) * width, out.dtype, "read").view(-1, width)
                acc[sel] += buf[rows].to(acc.dtype)
        out.copy_(acc)

    def allreduce_two_shot(self, src, dst, me, n, flags, counter, max_spins, status):
        self._wait(flags, len(src), int(counter), status)
        chunk = -(-n // len(src))
        chunk = -(-chunk // 4) * 4
        lo, hi = me * chunk, min((me + 1) * chunk, n)
        if hi <= lo:
            return
        acc = torch.zeros(hi - lo, dtype=torch.float32)
        for p in src:
            acc += self._typed(int(p) + 4 * lo, hi - lo, torch.float32, "read")
        for p in dst:
            self._typed(int(p) + 4 * lo, hi - lo, torch.float32, "write").copy_(acc)


class HostSymmetricHeap(SymmetricHeap):
    """Symmetric heap between the CPU ranks of one machine.  Construct it collectively (every rank, same size) after
    ``init_process_group``; it installs :class:`HostExt` as this process's native module, so use it only in processes that
    run no device kernels."""

    host = True

    def __init__(self, bytes_=64 << 20, wait_seconds=20.0, record=False):
        if not dist.is_initialized():
            raise RuntimeError("the symmetric heap needs an initialised process group (handle exchange)")
        self.device = torch.device("cpu")
        e = HostExt(dist.get_rank(), wait_seconds)
        if record:
            e.log = []
        native._EXT[0] = e
        self._map_heaps(e, bytes_)

    def check_recorded(self):
        """Collective over all ranks (heap built with ``record=True``): gather what every rank did to shared memory (accesses with
        their byte ranges, signals, barriers, waits) and run the happens-before check of :mod:`gt_b200.utils.hb_check` on the
        recorded programs.  Raises ``RuntimeError`` listing accesses that no chain of signals and waits orders (a read that could
        run before the write it follows in this run, a write that could land while a peer still reads).  Returns the report."""
        from ..utils.hb_check import check, trace_from_logs
        e = native.ext()
        logs = [None] * self.world
        dist.all_gather_object(logs, list(e.log))
        rep = check(trace_from_logs(logs), require_writes=False)
        if rep.violations or rep.expired or not rep.completed:
            lines = [f"{v.kind}: rank {v.rank}, memory of rank {v.owner} at offset {v.buf}: {v.detail}" for v in rep.violations[:8]]
            lines += [f"wait of rank {r} on flag {chan} for rank {peer} can never pass" for r, _, chan, peer in rep.expired[:8]]
            raise RuntimeError("recorded run of the peer-memory transport is not ordered by its signals and waits:\n  " + "\n  ".join(lines))
        return rep
