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
