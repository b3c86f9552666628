"""Happens-before checker for the peer-memory protocols (epoch channels, group barriers, staging buffers).

The kernels of this package order their accesses to other GPUs' memory with monotone epoch flags: ``signal`` publishes "my k-th
use of this channel is complete" to every member of a group, a consumer waits until the members it reads from have published
the epoch of its own latest signal (``gt_b200/csrc/p2p.cu``: ``channel_signal_kernel``, ``block_wait_channel``,
``barrier_kernel``).  Whether a buffer may be rewritten at some point of the program therefore depends on chains of such waits,
sometimes across several channels and groups.  This module checks those chains mechanically, on the CPU, for a symbolic
program of every rank:

* every rank's program is a straight line of ``write`` / ``read`` / ``signal`` / ``wait`` operations on named buffers and
  channels (no data-dependent control flow, one stream per rank), so the set of orderings that hold in EVERY execution is the
  happens-before relation "program order + (k-th signal of a peer -> the wait that needs epoch k)";
* vector clocks computed along one execution give exactly that relation; two conflicting accesses to a buffer (one of them a
  write) that it does not order are reported: a read that may run before the write it needs (``read-before-write``), a write
  that may overwrite data a peer is still reading (``write-while-read``), two unordered writes (``write-write``), and a read
  that finds another version than the one it names (``wrong-version``);
* faults are injected on the host side of the model: a signal that is never published, a rank that stops.  A wait nobody can
  satisfy then *expires*, as the bounded device waits do: the rank records ``100 + index of the silent peer`` in its status word
  and carries on, so the checker also shows that no rank can block for ever and which peer every status word names.

Two sources of programs: hand-written models (:mod:`gt_b200.parallel.protocol_model`) and recorded runs of the real code on the
host transport (:func:`trace_from_logs`, used by ``HostSymmetricHeap.check_recorded``).

The reference has no counterpart (its collectives are NCCL calls; ``gt3d/gt3d/dist/grid2d.py:55-69`` orders them with host
synchronisation); compute-sanitizer's race detection is the tool one would use on a device, this is the protocol-level
equivalent that needs none.
"""
import bisect
from collections import namedtuple

Violation = namedtuple("Violation", "kind rank op owner buf detail")
Report = namedtuple("Report", "violations status expired completed n_ops")


class ProtocolTrace:
    """Symbolic programs of ``world`` ranks.  ``buf`` and ``chan`` are hashable names; a buffer lives in the memory of ``owner``."""

    def __init__(self, world):
        self.world = int(world)
        self.prog = [[] for _ in range(self.world)]

    def write(self, rank, owner, buf, tag, note=""):
        self.prog[rank].append(("write", owner, buf, tag, note))

    def read(self, rank, owner, buf, tag, note=""):
        self.prog[rank].append(("read", owner, buf, tag, note))

    def signal(self, rank, chan, members, note=""):
        """``rank`` bumps its epoch on ``chan`` and publishes it to every rank of ``members``."""
        self.prog[rank].append(("signal", (chan, tuple(members)), None, None, note))

    def wait(self, rank, chan, members, peer, note=""):
        """Bounded wait until ``peer`` has published the epoch of ``rank``'s own latest signal on ``chan``."""
        self.prog[rank].append(("wait", (chan, tuple(members)), peer, None, note))

    def barrier(self, rank, chan, members, note=""):
        self.signal(rank, chan, members, note)
        for p in members:
            self.wait(rank, chan, members, p, note)

    def n_ops(self):
        return sum(len(p) for p in self.prog)


def check(trace, drop=(), die=None, max_violations=64, cascade=False, require_writes=True):
    """Run the programs of ``trace`` and return a :class:`Report`.

    ``drop``: set of ``(rank, chan, k)``: the k-th signal (1-based) of ``rank`` on channel name ``chan`` is not published.
    ``die``: dict ``rank -> op index``: the rank executes nothing from that operation on.
    ``cascade``: what happens when no rank can move.  ``False``: only the waits whose peer will never publish (its signal was
    dropped, or it has stopped) expire, and the ranks behind them carry on: the smallest set of expired waits, which names the
    root cause.  ``True``: every pending wait expires at once, as when all ranks started to wait at about the same time and
    run into the same limit together: the largest set.
    ``require_writes``: report a read of a location nobody has written.  Recorded runs (:func:`trace_from_logs`) switch it off:
    writes made by code outside the recorded entry points are not in the log."""
    world = trace.world
    die = dict(die or {})
    drop = set(drop)
    vc = [[0] * world for _ in range(world)]
    pc = [0] * world
    count = [dict() for _ in range(world)]                 # rank -> channel -> signals issued
    published = [dict() for _ in range(world)]             # rank -> channel -> sorted epochs that were published
    snap = {}                                              # (rank, channel, epoch) -> vector clock of the signal
    last_write = {}                                        # (owner, buf) -> (tag, writer, clock of the writer, op index)
    reads = {}                                             # (owner, buf) -> {reader: clock of the reader}
    violations, expired = [], []
    status = [0] * world

    def ordered(rank_a, clock_a, rank_b):                  # "the access of a at clock_a happens before b's current operation"
        return clock_a <= vc[rank_b][rank_a]

    def report(kind, rank, owner, buf, detail):
        if len(violations) < max_violations:
            violations.append(Violation(kind, rank, pc[rank], owner, buf, detail))

    def live(r):
        return pc[r] < len(trace.prog[r]) and not (r in die and pc[r] >= die[r])

    def silent(r):
        """The pending wait of rank r is on a peer that will never publish the epoch: the signal was issued and lost, or the peer
        has stopped (or finished) before issuing it."""
        op, chan, peer, _, _ = trace.prog[r][pc[r]]
        return op == "wait" and (count[peer].get(chan, 0) >= count[r].get(chan, 0) or not live(peer))

    def step(r, expire=False):
        """Execute the next operation of rank r; returns False if it is a wait that cannot pass yet."""
        op, a, b, tag, note = trace.prog[r][pc[r]]
        if op == "wait":
            chan, peer = a, b
            want = count[r].get(chan, 0)
            epochs = [k for k in published[peer].get(chan, ()) if k >= want]
            if want > 0 and not epochs:
                if not expire:
                    return False
                members = chan[1]
                status[r] = 100 + members.index(peer)
                expired.append((r, pc[r], chan[0], peer))
                vc[r][r] += 1
                pc[r] += 1
                return True
            vc[r][r] += 1
            if want > 0:
                s = snap[(peer, chan, min(epochs))]        # the earliest publication that satisfies the wait: the weakest guarantee
                for i in range(world):
                    if s[i] > vc[r][i]:
                        vc[r][i] = s[i]
            pc[r] += 1
            return True
        vc[r][r] += 1
        if op == "signal":
            chan = a
            k = count[r].get(chan, 0) + 1
            count[r][chan] = k
            if (r, chan[0], k) not in drop:
                published[r].setdefault(chan, []).append(k)
                snap[(r, chan, k)] = list(vc[r])
        elif op == "write":
            key = (a, b)
            lw = last_write.get(key)
            if lw is not None and lw[1] != r and not ordered(lw[1], lw[2], r):
                report("write-write", r, a, b, f"{note}: write of {tag} is not ordered after rank {lw[1]}'s write of {lw[0]}")
            for reader, c in reads.get(key, {}).items():
                if reader != r and not ordered(reader, c, r):
                    report("write-while-read", r, a, b, f"{note}: write of {tag} may overwrite {lw[0] if lw else None} while rank {reader} reads it")
            last_write[key] = (tag, r, vc[r][r], pc[r])
            reads[key] = {}
        elif op == "read":
            key = (a, b)
            lw = last_write.get(key)
            if lw is None:
                if require_writes:
                    report("read-before-write", r, a, b, f"{note}: nothing has been written where {tag} is expected")
            elif lw[1] != r and not ordered(lw[1], lw[2], r):
                report("read-before-write", r, a, b, f"{note}: read of {tag} is not ordered after rank {lw[1]}'s write of {lw[0]}")
            elif tag is not None and lw[0] != tag:
                report("wrong-version", r, a, b, f"{note}: expected {tag}, the buffer holds {lw[0]}")
            reads.setdefault(key, {})[r] = vc[r][r]
        pc[r] += 1
        return True

    while True:
        progressed = False
        for r in range(world):
            while live(r) and step(r):
                progressed = True
        if progressed:
            continue
        blocked = [r for r in range(world) if live(r)]
        if not blocked:
            break
        roots = [] if cascade else [r for r in blocked if silent(r)]
        for r in (roots or blocked):                       # nobody can move: pending waits run into their limit
            step(r, expire=True)
    completed = all(pc[r] >= len(trace.prog[r]) for r in range(world) if r not in die)
    return Report(violations, status, expired, completed, trace.n_ops())


def trace_from_logs(logs):
    """A :class:`ProtocolTrace` from what the ranks of a run on the host transport recorded (``HostExt.log`` of every rank, in rank
    order): events ``(kind, owner, offset, bytes)`` for ``kind`` in view / write / read, ``("signal", flag offset, members)``,
    ``("barrier", flag offset, members)`` and ``("wait", flag offset, member index)``.

    Byte ranges are cut at every boundary that occurs in the logs of the same owner, so overlapping accesses meet on common
    pieces.  A ``view`` (a tensor over heap memory handed to code outside the recorded entry points) counts as a write of its
    range unless the next recorded event of that rank (waits aside) is an access that starts at the same address: then the view
    was only the operand of that access.  Reads name no version (``tag=None``)."""
    world = len(logs)
    events = []
    for r, log in enumerate(logs):
        out = []
        for i, ev in enumerate(log):
            if ev[0] == "view":
                j = i + 1
                while j < len(log) and log[j][0] == "wait":          # a kernel waits before it touches its operand
                    j += 1
                nxt = log[j] if j < len(log) else None
                if nxt is not None and nxt[0] in ("read", "write") and nxt[1] == ev[1] and nxt[2] == ev[2]:
                    continue
                ev = ("write",) + tuple(ev[1:])
            out.append(ev)
        events.append(out)
    cuts = {}
    for log in events:
        for ev in log:
            if ev[0] in ("read", "write"):
                cuts.setdefault(ev[1], set()).update((ev[2], ev[2] + ev[3]))
    cuts = {o: sorted(c) for o, c in cuts.items()}
    tr = ProtocolTrace(world)
    for r, log in enumerate(events):
        members_of = {}
        for ev in log:
            if ev[0] in ("read", "write"):
                c = cuts[ev[1]]
                i, j = bisect.bisect_left(c, ev[2]), bisect.bisect_left(c, ev[2] + ev[3])
                for lo in c[i:j]:
                    (tr.write if ev[0] == "write" else tr.read)(r, ev[1], lo, None, f"{ev[0]} of {ev[3]} bytes at offset {ev[2]}")
            elif ev[0] == "signal":
                members_of[ev[1]] = ev[2]
                tr.signal(r, ev[1], ev[2])
            elif ev[0] == "barrier":
                members_of[ev[1]] = ev[2]
                tr.barrier(r, ev[1], ev[2])
            elif ev[0] == "wait":
                members = members_of[ev[1]]
                tr.wait(r, ev[1], members, members[ev[2]])
    return tr
