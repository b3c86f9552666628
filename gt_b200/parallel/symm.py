"""Symmetric heap and peer-memory collectives (NVLink 5 / NVSwitch, one process per GPU).

Every rank ``cudaMalloc``s one heap of the same size, exports it with CUDA IPC and opens the heaps of the peers on its machine, so
every kernel can be given a table of peer base addresses.  A job on several machines keeps one heap per rank all the same; a
process group then runs on this transport if all of its ranks share a machine (``group_is_local``) and on NCCL otherwise.  Allocation inside the heap is a bump allocator that all
ranks drive with the same sequence of requests: an object therefore lives at the same offset on every rank
("symmetric").  NCCL / gloo is only used once, to exchange the 64-byte IPC handles.

Collectives are *receiver driven*: a rank publishes its contribution in a staging buffer of the heap, a group barrier
orders the publication, and the rank's own kernel then reads what it needs from the peers' buffers
(``csrc/p2p.cu``): dense all-gather / reduce-scatter / all-reduce, and the sparse ``pull_gather`` / ``pull_reduce`` that
move only the rows a tile references.  Reductions sum in fp32 in a fixed peer order.

Synchronisation.  One barrier per collective: a kernel that publishes a device-resident epoch into every peer's flag
array and waits (bounded) for the peers' epochs.  The epoch counter lives in device memory, so a captured CUDA graph
replays correctly.  Staging buffers are keyed by the position of the collective inside the step (``begin_step`` resets
the position and issues one extra barrier), so a buffer is rewritten only after at least one later barrier, which
implies that every peer has finished reading the previous contents.  A wait that expires writes the peer index to the
status word (``gt_b200.ops.native.check_status`` raises on the host); nothing spins forever.
"""
import os
import socket
import zlib

import torch
import torch.distributed as dist

from ..ops import native

_DT = {torch.float32: 0, torch.bfloat16: 1, torch.int32: 2, torch.int64: 3, torch.uint8: 4,
       torch.float64: 5}        # 5: host emulation only (parity tests in double precision); the device kernels move fp32 / bf16

# polls before a wait on a peer gives up (~1 s at the default).  A rank-local stall longer than this (first-launch module
# loading, a slow evaluation on one rank) makes the wait expire, so runs with long rank-local phases raise it.
MAX_SPINS = int(os.environ.get("GT_PEER_WAIT_SPINS", "5000000"))
# Eager steps (warm-up before a CUDA graph exists, tests, the first steps of a run) let the ranks' host code drift apart by whole
# seconds: first-launch module loading, plan construction, a new communicator.  A wait enqueued eagerly therefore gets a longer
# (still finite) limit than one recorded into a CUDA graph, whose launches are all enqueued at once.
MAX_SPINS_EAGER = int(os.environ.get("GT_PEER_WAIT_SPINS_EAGER", str(20 * MAX_SPINS)))


_NO_CUDA = [False]


def wait_spins():
    """Poll limit for a peer wait that is being enqueued now."""
    if _NO_CUDA[0]:
        return MAX_SPINS_EAGER
    try:
        capturing = torch.cuda.is_current_stream_capturing()
    except Exception:                                       # no CUDA runtime in this process: the host emulation of the heap
        _NO_CUDA[0] = True
        capturing = False
    return MAX_SPINS if capturing else MAX_SPINS_EAGER


def alloc_log_update(log, off, nbytes):
    """``(number of allocations, running CRC of their offsets and sizes)`` after one more allocation."""
    n, crc = log
    return n + 1, zlib.crc32(f"{off}:{nbytes};".encode(), crc)


def check_alloc_logs(log, group=None):
    """Compare the allocation logs of the ranks of ``group``; raises ``RuntimeError`` naming the ranks that differ."""
    world = dist.get_world_size(group)
    logs = [None] * world
    dist.all_gather_object(logs, tuple(log), group=group)
    if len(set(logs)) > 1:
        common = max(set(logs), key=logs.count)
        odd = [i for i, v in enumerate(logs) if v != common]
        raise RuntimeError(f"symmetric heap out of step: ranks {odd} of the group made a different sequence of allocations "
                           f"(allocations, checksum) = {logs}; every rank must allocate the same sizes in the same order")


class GroupContext:
    """Peers of one process group: index of this rank, global ranks, flag array and barrier counter."""

    def __init__(self, heap, group, name):
        self.heap, self.group, self.name = heap, group, name
        self.size = dist.get_world_size(group)
        self.me = dist.get_rank(group)
        self.ranks = [dist.get_global_rank(group, i) if group is not None else i for i in range(self.size)]
        self.flags_off = heap.alloc(4 * 64)                     # int32[64] epoch flags written by the peers
        self.flags = heap.view(self.flags_off, (64,), torch.int32)
        self.counter = torch.zeros(1, dtype=torch.int32, device=heap.device)
        self.peer_flag_ptrs = heap.peer_table(self.flags_off, self.ranks)
        self.kind_count = {}                                    # collectives of each kind issued since begin_step
        self.buffers = {}                                       # (kind, parity) -> (offset, nbytes)

    def barrier(self):
        native.ext().group_barrier(self.peer_flag_ptrs, self.flags, self.counter, self.me, wait_spins(), native.status(self.heap.device))

    def staging(self, nbytes, kind):
        """Staging buffer for the next collective of ``kind`` on this group (same offset on all ranks of the group).

        Two buffers per kind are used alternately.  Every collective here is "write the buffer, group barrier, peers read (or:
        peers write, barrier, owner reads)", so when a buffer comes up again two uses later, the barrier of the use in between
        has been passed by every peer after it finished with the buffer: two buffers per kind are enough however many layers
        a step has, and the heap does not grow with the depth of the model."""
        n = self.kind_count.get(kind, 0)
        self.kind_count[kind] = n + 1
        key = (kind, n & 1)
        buf = self.buffers.get(key)
        if buf is None or buf[1] < nbytes:
            buf = (self.heap.alloc(nbytes), nbytes)
            self.buffers[key] = buf
        return buf[0]


class SymmetricHeap:
    host = False                 # True in the host emulation (symm_host.HostSymmetricHeap): CPU tensors, float64 allowed

    def __init__(self, device, bytes_=1 << 30):
        if not dist.is_initialized():
            raise RuntimeError("the symmetric heap needs an initialised process group (IPC handle exchange)")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self._map_heaps(native.ext(), bytes_)

    def _map_heaps(self, e, bytes_):
        """Allocate this rank's heap, exchange the handles and map every peer's heap."""
        self.bytes = int(bytes_)
        self.base = e.heap_alloc(self.bytes)
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        handles = [None] * self.world
        # GT_HOSTNAME overrides the machine name (tests split the ranks of one machine into pretended nodes)
        dist.all_gather_object(handles, (self.rank, e.heap_ipc_handle(self.base), os.environ.get("GT_HOSTNAME") or socket.gethostname()))
        # Peer memory is mapped between the ranks of ONE machine.  When the process group covers several, every rank maps the heaps
        # of its own machine only: a group whose members all share a machine runs on the peer-memory transport, any other group
        # stays on NCCL (``group_is_local``), and every rank still makes the same allocations, so offsets agree wherever they are used.
        self.hosts = [None] * self.world
        for r, _, host in handles:
            self.hosts[r] = host
        self.peer_base = [0] * self.world
        for r, h, host in handles:
            if host == self.hosts[self.rank]:
                self.peer_base[r] = self.base if r == self.rank else e.heap_open(h)
        self._local_groups = {}
        per_host = {}
        for r, host in enumerate(self.hosts):
            per_host.setdefault(host, []).append(r)
        # groups of one kind are all local or all remote only if every machine holds the same number of consecutive ranks
        self.uniform_placement = len({len(v) for v in per_host.values()}) == 1 and all(v == list(range(v[0], v[0] + len(v))) for v in per_host.values())
        if not self.uniform_placement and self.rank == 0:
            print(f"[symm] ranks per machine {sorted(len(v) for v in per_host.values())}: groups of one kind may differ in transport between "
                  "ranks; check_symmetric() will tell whether the heaps stay in step", flush=True)
        self.top = 0
        self.alloc_log = (0, 0)
        self.groups = {}
        self.named = {}
        dist.barrier()

    # ---- allocation ------------------------------------------------------------------------------------------------------
    def alloc(self, nbytes, align=256):
        off = -(-self.top // align) * align
        if off + nbytes > self.bytes:
            raise MemoryError(f"symmetric heap exhausted: need {off + nbytes} bytes, have {self.bytes} (raise --heap_mb)")
        self.top = off + nbytes
        self.alloc_log = alloc_log_update(self.alloc_log, off, nbytes)
        return off

    def check_symmetric(self, group=None):
        """Raise unless every rank has made the same sequence of allocations (same offsets and sizes in the same order): peers
        address each other's buffers by offset, so one rank that allocates differently leaves everyone reading the wrong bytes
        and waiting on the wrong flags.  Collective over ``group`` (default: all ranks); host side only."""
        check_alloc_logs(self.alloc_log, group)

    def _float_types(self):
        return (torch.float32, torch.bfloat16, torch.float64) if self.host else (torch.float32, torch.bfloat16)

    def group_is_local(self, group=None):
        """Every rank of ``group`` (default: all ranks) runs on this rank's machine, so their heaps are mapped here."""
        key = id(group) if group is not None else None
        ok = self._local_groups.get(key)
        if ok is None:
            ranks = range(self.world) if group is None else dist.get_process_group_ranks(group)
            ok = self._local_groups[key] = all(self.hosts[r] == self.hosts[self.rank] for r in ranks)
        return ok

    def reaches(self, x, group=None):
        """``x`` lives where this heap's kernels run, and the heaps of all ranks of ``group`` are mapped on this rank."""
        return (x.is_cuda or self.host) and self.group_is_local(group)

    def view(self, off, shape, dtype):
        return native.ext().tensor_from_ptr(self.base + off, list(shape), _DT[dtype], self.device.index or 0)

    def empty(self, numel, dtype, name=None):
        """A tensor inside the heap (same offset on every rank when all ranks allocate in the same order)."""
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        off = self.alloc(nbytes)
        t = self.view(off, (numel,), dtype)
        if name is not None:
            self.named[name] = (off, nbytes)
        return t

    def peer_table(self, off, ranks):
        """int64 device tensor with the address of offset ``off`` in the heap of every rank of ``ranks``."""
        return torch.tensor([self.peer_base[r] + off for r in ranks], dtype=torch.int64, device=self.device)

    def ctx(self, group):
        key = id(group) if group is not None else None
        c = self.groups.get(key)
        if c is None:
            if not self.group_is_local(group):
                # never hand a kernel the address of a heap that is not mapped here: refuse on the host
                raise RuntimeError("this group crosses machines: its collectives run on NCCL, not on the peer-memory transport "
                                   "(callers test SymmetricHeap.group_is_local / reaches first)")
            c = self.groups[key] = GroupContext(self, group, str(key))
        return c

    def begin_step(self):
        """Call at the start of every step (before capture / replay): restarts the alternation of the staging buffers, so that
        every step (eager, captured or replayed) uses the same offsets, and synchronises the groups."""
        for c in self.groups.values():
            c.kind_count.clear()
            c.barrier()

    # ---- dense collectives ------------------------------------------------------------------------------------------------
    def all_gather(self, x, group):
        c = self.ctx(group)
        x = x.contiguous()
        nbytes = x.numel() * x.element_size()
        if nbytes % 16:
            raise ValueError("all_gather payload must be a multiple of 16 bytes per rank")
        off = c.staging(nbytes, "ag")
        self.view(off, x.shape, x.dtype).copy_(x)
        c.barrier()
        out = torch.empty((c.size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        native.ext().pull_all_gather(self.peer_table_cached(c, off), out)
        return out

    def reduce_scatter(self, x, group):
        c = self.ctx(group)
        x = x.contiguous()
        if x.dtype not in self._float_types() or (x.numel() // c.size) % 8:
            raise ValueError("reduce_scatter needs fp32 / bf16 chunks that are multiples of 8 elements")
        nbytes = x.numel() * x.element_size()
        off = c.staging(nbytes, "rs")
        self.view(off, x.shape, x.dtype).copy_(x)
        c.barrier()
        out = torch.empty((x.shape[0] // c.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        native.ext().pull_reduce_scatter(self.peer_table_cached(c, off), c.me, out)
        return out

    # ---- collectives fused into the tensor-core GEMMs ------------------------------------------------------------------------
    def linear_gather(self, x, w, group, bias=None, act=None, want_gathered=True):
        """``all_gather(x) @ w^T`` in one kernel: the GEMM's TMA loads read each rank's ``x [chunk, K]`` (bf16) from the
        owner's heap, tile by tile.  Returns ``(y [G * chunk, N], gathered x or None)``."""
        c = self.ctx(group)
        x = x.contiguous()
        chunk, k = x.shape
        off = c.staging(x.numel() * 2, "agg")
        self.view(off, x.shape, torch.bfloat16).copy_(x)
        c.barrier()                                               # every rank's x is in place
        y = torch.empty(c.size * chunk, w.shape[0], dtype=torch.bfloat16, device=x.device)
        xg = torch.empty(c.size * chunk, k, dtype=torch.bfloat16, device=x.device) if want_gathered else None
        native.ext().gemm_nt_gather([self.peer_base[r] + off for r in c.ranks], chunk, k, k, w, y, bias, {None: 0, "relu": 1, "gelu": 2}[act],
                                    0.0, None, 0, xg, native.status(self.device), None, None, 0, 0)
        return y, xg

    def linear_scatter(self, a, w, group, out_dtype=torch.bfloat16, out=None, accumulate=False):
        """``reduce_scatter(a @ w^T)`` with the scatter in the GEMM epilogue: finished tiles are stored straight into the
        owning rank's heap; after a barrier the owner adds the ``G`` slots.  ``a [G * chunk, K]``, ``w [N, K]`` bf16."""
        c = self.ctx(group)
        chunk, n = a.shape[0] // c.size, w.shape[0]
        slot = chunk * n * 2
        off = c.staging(c.size * slot, "grs")
        native.ext().gemm_nt_scatter(a, w, [self.peer_base[r] + off + c.me * slot for r in c.ranks], chunk, n, native.status(self.device))
        c.barrier()                                               # every rank's tiles have landed in my slots
        if out is None:
            out = torch.empty(chunk, n, dtype=out_dtype, device=a.device)
            accumulate = False
        native.ext().sum_slots(self.view(off, (c.size, chunk, n), torch.bfloat16), out, accumulate)
        return out

    def publish(self, x, group, kind="pub"):
        """Copy ``x`` into this call site's staging buffer and return ``(offset, int64 device table of the peers' addresses)``
        after a barrier: every rank of the group may then read every rank's ``x`` in place."""
        c = self.ctx(group)
        x = x.contiguous()
        off = c.staging(x.numel() * x.element_size(), kind)
        self.view(off, x.shape, x.dtype).copy_(x)
        c.barrier()
        return off, self.peer_table_cached(c, off)

    def rows_to_heads(self, x, group):
        """Ulysses all-to-all ``[chunk, H, d] -> [P * chunk, H / P, d]`` by strided peer reads (no transposed staging copies)."""
        c = self.ctx(group)
        chunk, h, d = x.shape
        slab = (h // c.size) * d * x.element_size()
        _, table = self.publish(x, group, "a2a_h")
        out = torch.empty(c.size * chunk, h // c.size, d, dtype=x.dtype, device=x.device)
        native.ext().pull_all_to_all(table, c.me, chunk, slab, True, out)
        return out

    def heads_to_rows(self, y, group):
        """Inverse: ``[P * chunk, H / P, d] -> [chunk, H, d]``."""
        c = self.ctx(group)
        n, hg, d = y.shape
        chunk = n // c.size
        slab = hg * d * y.element_size()
        _, table = self.publish(y, group, "a2a_r")
        out = torch.empty(chunk, c.size * hg, d, dtype=y.dtype, device=y.device)
        native.ext().pull_all_to_all(table, c.me, chunk, slab, False, out)
        return out

    def all_reduce(self, x, out, name=None, group=None):
        """``out = sum over ranks of x``; ``x`` should live in the heap (``heap.empty``), otherwise it is staged."""
        c = self.ctx(group)
        if name is not None and name in self.named:
            off = self.named[name][0]
        else:
            off = c.staging(x.numel() * x.element_size(), "ar")
            self.view(off, x.shape, x.dtype).copy_(x)
        c.barrier()
        native.ext().pull_all_reduce(self.peer_table_cached(c, off), out)
        c.barrier()                      # x (the gradient buffer) is rewritten right away by the next step's zero-fill
        return out

    def all_reduce_two_shot(self, name, out_name, n, group=None):
        """Sum of the heap tensor ``name`` (fp32, ``heap.empty(..., name)``) over the group into the heap tensor ``out_name`` on every
        member: each rank reduces one slice from all members and stores it to all members; ordering by two epoch channels (no
        barrier).  Returns after enqueueing; the result is complete on this rank once the second channel's wait has passed."""
        from .fused_layer import Channel
        c = self.ctx(group)
        key = ("ar2", name, out_name)
        st = c.buffers.get(key)
        if st is None:
            st = c.buffers[key] = (Channel(self, c), Channel(self, c))
        ready, done = st
        src, dst = self.named[name][0], self.named[out_name][0]
        e = native.ext()
        status = native.status(self.device)
        ready.signal()                                            # my contribution is final
        e.allreduce_two_shot([self.peer_base[r] + src for r in c.ranks], [self.peer_base[r] + dst for r in c.ranks], c.me, n,
                             ready.flags, ready.counter, wait_spins(), status)
        done.signal()                                             # my slice has been stored everywhere
        e.channel_wait(done.flags, done.counter, c.size, wait_spins(), status)

    def peer_table_cached(self, c, off):
        key = ("tbl", off)
        t = c.buffers.get(key)
        if t is None:
            t = c.buffers[key] = self.peer_table(off, c.ranks)
        return t

    # ---- sparse collectives (SparseRowPlan transports) -----------------------------------------------------------------------
    def _plan_state(self, plan):
        st = getattr(plan, "_pull", None)
        if st is None:
            c = self.ctx(plan.group)
            # owner-side table of the reduce: for every peer p and owned row r, the compact row of p that holds a partial of r
            dev = self.device
            src = torch.full((c.size, plan.rows_per_rank), -1, dtype=torch.int32, device=dev)
            send = torch.stack([self._compact_index_for(plan, p, dev) for p in range(c.size)]).contiguous()
            dist.all_to_all_single(src, send, group=plan.group)          # row p of src: peer p's compact rows for my rows
            # staging rows of the reduce: the largest need set of ANY rank, so that every rank's heap grows by the same amount
            st = plan._pull = dict(ctx=c, src=src.contiguous(), n_max=int(plan.n_need_max))
        return st

    @staticmethod
    def _compact_index_for(plan, p, dev):
        """For owner ``p``: compact row (in my need set) of each of p's rows, -1 where I hold no partial."""
        out = torch.full((plan.rows_per_rank,), -1, dtype=torch.int32, device=dev)
        sel = plan.need_owner == p
        out[plan.need_row[sel].long()] = torch.nonzero(sel).squeeze(1).to(torch.int32)
        return out

    def pull_gather(self, x2, plan):
        """``x2 [rows_per_rank, F]`` (my chunk) -> ``[n_need, F]``: the rows of the block this rank's tile references."""
        st = self._plan_state(plan)
        c = st["ctx"]
        nbytes = x2.numel() * x2.element_size()
        if (x2.shape[1] * x2.element_size()) % 16:
            raise ValueError("rows must be a multiple of 16 bytes")
        off = c.staging(nbytes, "pg")
        self.view(off, x2.shape, x2.dtype).copy_(x2)
        c.barrier()
        out = torch.empty(plan.n_need, x2.shape[1], dtype=x2.dtype, device=x2.device)
        native.ext().pull_gather_rows(self.peer_table_cached(c, off), plan.need_owner, plan.need_row, out)
        return out

    def pull_reduce(self, y2, plan):
        """``y2 [n_need, F]`` partial rows -> ``[rows_per_rank, F]``: sum of the partials the peers hold for my rows."""
        st = self._plan_state(plan)
        c = st["ctx"]
        if y2.shape[1] % 8 or y2.dtype not in self._float_types():
            raise ValueError("pull_reduce needs fp32 / bf16 rows with a width that is a multiple of 8")
        nbytes = max(st["n_max"], 1) * y2.shape[1] * y2.element_size()
        off = c.staging(nbytes, "pr")
        if plan.n_need:
            self.view(off, y2.shape, y2.dtype).copy_(y2)
        c.barrier()
        out = torch.empty(plan.rows_per_rank, y2.shape[1], dtype=y2.dtype, device=y2.device)
        native.ext().pull_reduce_rows(self.peer_table_cached(c, off), st["src"], out)
        return out

    def close(self):
        e = native.ext()
        for r, p in enumerate(self.peer_base):
            if r != self.rank and p:
                e.heap_close(p)
        e.heap_free(self.base)


def selftest():
    """``torchrun --nproc-per-node N -m gt_b200.parallel.symm``: heap set-up, IPC mapping, barrier and one collective of
    each kind against NCCL (the role of the reference's ``gt3d/gt3d/dist/pullcomm/selftest.cu``)."""
    import os
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    heap = SymmetricHeap(dev, 64 << 20)
    ok = True
    for rep in range(3):
        heap.begin_step()
        x = torch.full((1024, 16), float(rank + rep), device=dev)
        ref = torch.empty(world * 1024, 16, device=dev)
        dist.all_gather_into_tensor(ref, x)
        ok &= bool(torch.equal(heap.all_gather(x, None), ref))
        y = torch.randn(world * 256, 16, device=dev)
        ref = torch.empty(256, 16, device=dev)
        dist.reduce_scatter_tensor(ref, y)
        ok &= bool((heap.reduce_scatter(y, None) - ref).abs().max() < 1e-4)
    torch.cuda.synchronize()
    native.check_status(dev)
    flag = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"symmetric heap selftest on {world} GPUs: {'ALL PASSED' if int(flag) else 'FAILED'}", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0 if int(flag) else 1)


if __name__ == "__main__":
    selftest()
