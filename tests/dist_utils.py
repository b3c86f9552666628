"""Spawn ``world`` CPU ranks on the gloo backend and run ``fn(rank, world, *args)`` in each; any exception fails the test."""
import os
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _entry(rank, world, path, fn, args, err_q):
    try:
        torch.set_num_threads(1)
        dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
        fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        err_q.put((rank, traceback.format_exc()))
        raise


def run_dist(fn, world, *args, timeout=300):
    ctx = mp.get_context("spawn")
    err_q = ctx.SimpleQueue()
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "store")
        procs = [ctx.Process(target=_entry, args=(r, world, path, fn, args, err_q)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout)
        bad = [p for p in procs if p.is_alive() or p.exitcode != 0]
        for p in procs:
            if p.is_alive():
                p.terminate()
        if bad:
            msgs = []
            while not err_q.empty():
                msgs.append("rank %d:\n%s" % err_q.get())
            raise AssertionError("distributed test failed\n" + "\n".join(msgs))


def _group_entry(rank, world, fn, cases, done_path):
    """All cases of one world size in ONE set of processes (a process start costs more than a case); rank 0 notes every case that
    all ranks finished, so that the test of a case can tell whether it ran, failed or was never reached."""
    for case in cases:
        try:
            fn(rank, world, case)
        except Exception as exc:
            raise AssertionError(f"case {case}: {type(exc).__name__}: {exc}") from exc
        dist.barrier()
        if rank == 0:
            with open(done_path, "a") as f:
                f.write(case + "\n")


_GROUPS = {}


def grouped_case(fn, cases, world, case, timeout=1200):
    """Assert that ``case`` passed in the grouped run of ``cases`` (all of world size ``world``) through ``fn(rank, world, case)``; the
    group runs once per test session."""
    key = (fn.__module__, fn.__name__, world)
    if key not in _GROUPS:
        with tempfile.TemporaryDirectory() as tmp:
            done = os.path.join(tmp, "done")
            open(done, "w").close()
            err = None
            try:
                run_dist(_group_entry, world, fn, list(cases), done, timeout=timeout)
            except AssertionError as exc:
                err = str(exc)
            _GROUPS[key] = (set(open(done).read().split()), err)
    ok, err = _GROUPS[key]
    assert case in ok, err or f"case {case} did not run"
