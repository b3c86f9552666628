"""Failure detection without faulting anything: failures are made on the host (a rank that raises, leaves or goes silent;
a corrupted plan) and, on a GPU, by a bounded wait on a flag that nothing sets."""
import os
import time

import pytest
import torch

from dist_utils import run_dist


def _heartbeat_worker(rank, world, mode):
    import torch.distributed as dist
    from gt_b200.utils.health import Heartbeat, PeerFailure
    hb = Heartbeat(timeout=1.0)
    dist.barrier()
    if mode == "leaves":
        if rank == 1:
            hb.leave()                                          # between steps, nothing in flight
        dist.barrier()
        if rank != 1:
            with pytest.raises(PeerFailure) as e:
                hb.check()
            assert e.value.ranks == [1] and "left" in str(e.value)
    elif mode == "raises":
        def step():
            if rank == 2:
                raise ValueError("loss is not finite")
            return 1
        if rank == 2:
            with pytest.raises(ValueError):
                hb.guarded(step)
        else:
            assert hb.guarded(step) == 1
        dist.barrier()
        if rank != 2:
            with pytest.raises(PeerFailure) as e:
                hb.check()
            assert e.value.ranks == [2] and "ValueError" in str(e.value)
    else:                                                       # "silent": rank 0 stops beating
        for _ in range(3):
            if rank != 0:
                hb.beat()
            hb.check() if rank == 0 else None
            time.sleep(0.1)
        if rank != 0:
            hb.check()                                          # first look records the counters
            t0 = time.monotonic()
            with pytest.raises(PeerFailure) as e:
                while time.monotonic() - t0 < 10:
                    hb.beat()
                    hb.check()
                    time.sleep(0.2)
            assert e.value.ranks == [0] and "silent" in str(e.value)
        else:
            time.sleep(2.5)
    dist.barrier()


@pytest.mark.parametrize("mode", ["leaves", "raises", "silent"])
def test_heartbeat_reports_dead_peers(mode):
    run_dist(_heartbeat_worker, 3, mode)


def _timeout_worker(rank, world, store_path):
    """A rank that never joins a collective: the others' collective ends with an error after the group's short timeout."""
    import datetime
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method=f"file://{store_path}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=3))
    x = torch.ones(4)
    dist.all_reduce(x)                                          # everyone takes part: fine
    if rank == 1:
        os._exit(0)                                             # leaves between steps
    t0 = time.monotonic()
    try:
        dist.all_reduce(x)
        ok = False
    except Exception:
        ok = True
    assert ok and time.monotonic() - t0 < 30
    os._exit(0)


def test_collective_with_a_missing_rank_times_out(tmp_path):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_timeout_worker, args=(r, 2, str(tmp_path / "store"))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    assert all((not p.is_alive()) and p.exitcode == 0 for p in procs)


def test_corrupted_structures_are_caught_on_the_host():
    from gt_b200.attention import BlockCSR
    from gt_b200.utils.checks import StructureError, validate_block, validate_segment_plan
    ei = torch.randint(0, 50, (2, 400))
    et = torch.randint(0, 3, (400,))
    blk = BlockCSR.from_edges(ei, 50, 50, et)
    assert validate_block(blk, num_types=3)
    plan = blk.row_plan(16)
    assert validate_segment_plan(plan, 50, 400)
    bad = BlockCSR.from_edges(ei, 50, 50, et)
    bad.col[7] = 50                                             # one past the column block
    with pytest.raises(StructureError, match="outside the column block"):
        validate_block(bad, 3)
    bad = BlockCSR.from_edges(ei, 50, 50, et)
    bad.crow[10] = bad.crow[9] - 1
    with pytest.raises(StructureError):
        validate_block(bad, 3)
    with pytest.raises(StructureError, match="edge type"):
        validate_block(blk, num_types=2)
    plan.seg_end[0] = 401
    with pytest.raises(StructureError, match="edge range"):
        validate_segment_plan(plan, 50, 400)


@pytest.mark.gpu
def test_bounded_device_wait_expires_and_the_context_survives():
    """A barrier whose peer never arrives: the wait runs out after a few thousand polls, the status word says which peer
    was missing, and the device keeps working."""
    from gt_b200.ops import native
    dev = torch.device("cuda:0")
    e = native.ext()
    flags = torch.zeros(64, dtype=torch.int32, device=dev)              # my flags: nobody will ever write slot 1
    other = torch.zeros(64, dtype=torch.int32, device=dev)              # the "peer's" flags live on this GPU too
    table = torch.tensor([flags.data_ptr(), other.data_ptr()], dtype=torch.int64, device=dev)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    native.status(dev).zero_()
    e.group_barrier(table, flags, counter, 0, 2000, native.status(dev))
    torch.cuda.synchronize()
    code = int(native.status(dev).item())
    assert code >= 100, code                                            # 100 + index of the silent peer
    with pytest.raises(RuntimeError, match="expired wait"):
        native.check_status(dev)
    assert int(native.status(dev).item()) == 0                          # cleared by the check
    x = torch.arange(8, device=dev).float()
    assert float((x * 2).sum()) == 56.0                                 # the context is alive
    assert int(other[0].item()) != 0                                    # my arrival was published before the wait


def _alloc_log_worker(rank, world):
    """Allocation logs that agree pass; a rank that allocated a different size is named."""
    from gt_b200.parallel.symm import alloc_log_update, check_alloc_logs
    log = (0, 0)
    for off, nbytes in ((0, 256), (256, 4096), (4352, 32)):
        log = alloc_log_update(log, off, nbytes)
    check_alloc_logs(log)                                   # identical on every rank
    bad = alloc_log_update(log, 4608, 1024 if rank != 2 else 2048)
    try:
        check_alloc_logs(bad)
    except RuntimeError as exc:
        assert "ranks [2]" in str(exc)
    else:
        raise AssertionError("a rank with a different allocation went unnoticed")


def test_symmetric_heap_allocation_logs_are_compared_across_ranks():
    from dist_utils import run_dist
    run_dist(_alloc_log_worker, 4)


def test_every_polling_loop_in_the_kernel_sources_is_bounded():
    """Source check of the rule that no device wait may spin for ever: every ``while`` loop that polls a peer flag, an mbarrier or an
    asynchronous-copy group names a limit (a spin count or a clock budget) in its condition or in the lines right below it."""
    import glob
    import os
    import re
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "gt_b200", "csrc")
    poll = re.compile(r"while\s*\(.*(ld_acquire|try_wait|test_wait|volatile|ld_relaxed|\*flag|->flag)")
    bound = re.compile(r"spins|kWaitCycles|clock64|tries|max_iter|limit", re.I)
    found, unbounded = 0, []
    for path in sorted(glob.glob(os.path.join(root, "*.cu")) + glob.glob(os.path.join(root, "*.cuh")) + glob.glob(os.path.join(root, "*.h"))):
        lines = open(path).read().splitlines()
        for i, line in enumerate(lines):
            if poll.search(line) and not line.lstrip().startswith("//"):
                found += 1
                if not bound.search(" ".join(lines[i:i + 4])):
                    unbounded.append((os.path.basename(path), i + 1, line.strip()))
    assert found >= 12, found
    assert not unbounded, unbounded
