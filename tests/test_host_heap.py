"""The peer-memory transport between CPU processes (``gt_b200.parallel.symm_host``): the production heap logic on shared host memory,
checked against gloo, on grids with two non-trivial axes."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_dist  # noqa: E402


def _collectives_worker(rank, world, dtype_name):
    import torch.distributed as dist
    from gt_b200.ops import native
    from gt_b200.parallel.grid import make_grid
    from gt_b200.parallel.sparse_comm import SparseRowPlan
    from gt_b200.parallel.symm_host import HostSymmetricHeap
    dtype = getattr(torch, dtype_name)
    tol = dict(float64=1e-12, float32=1e-5, bfloat16=5e-2)[dtype_name]
    grid = make_grid((2, 2), 64, n_pad=64)
    heap = HostSymmetricHeap(8 << 20, wait_seconds=30.0)
    g = torch.Generator().manual_seed(100 + rank)
    try:
        for rep in range(3):                                 # three rounds: every staging copy is reused
            heap.begin_step()
            for group in (grid.row_group, grid.col_group, None):
                size = dist.get_world_size(group)
                me = dist.get_rank(group)
                x = torch.randn(24, 16, generator=g).to(dtype)
                ref = [torch.empty_like(x) for _ in range(size)]
                dist.all_gather(ref, x, group=group)
                assert torch.equal(heap.all_gather(x, group), torch.cat(ref)), "all_gather"
                y = torch.randn(size * 8, 16, generator=g).to(dtype)
                tot = y.double().clone()
                dist.all_reduce(tot, group=group)
                got = heap.reduce_scatter(y, group)
                assert (got.double() - tot[me * 8:(me + 1) * 8]).abs().max() < tol * size, "reduce_scatter"
                z = torch.randn(40, generator=g).to(dtype)
                tot = z.double().clone()
                dist.all_reduce(tot, group=group)
                assert (heap.all_reduce(z, torch.empty_like(z), group=group).double() - tot).abs().max() < tol * size, "all_reduce"
                h = torch.randn(6, 2 * size, 8, generator=g).to(dtype)            # Ulysses all-to-all, there and back
                t = heap.rows_to_heads(h, group)
                send = h.view(6, size, 2, 8).transpose(0, 1).contiguous()
                recv = torch.empty_like(send)
                dist.all_to_all_single(recv, send, group=group)
                assert torch.equal(t, recv.view(size * 6, 2, 8)), "rows_to_heads"
                assert torch.equal(heap.heads_to_rows(t, group), h), "heads_to_rows"
            # sparse plans whose need sets differ between the two row groups (3 rows against 29) and between the members of a group
            per = grid.n_row_block // 2
            n_need = (3 if grid.r == 0 else 29) + grid.c
            need = torch.randperm(2 * per, generator=torch.Generator().manual_seed(7 + rank))[:n_need].sort().values
            plans = {t: SparseRowPlan(grid.row_group, per, need, "row", t, heap if t == "pull" else None) for t in ("a2a", "pull")}
            x = torch.randn(per, 16, generator=g).to(dtype)
            assert torch.equal(plans["pull"].gather(x), plans["a2a"].gather(x)), "sparse gather"
            y = torch.randn(n_need, 16, generator=g).to(dtype)
            a, b = plans["pull"].reduce_scatter(y), plans["a2a"].reduce_scatter(y)
            assert (a.double() - b.double()).abs().max() < tol * 2, "sparse reduce_scatter"
            # a collective of the COLUMN group right after the row groups grew their heaps: the offsets must still agree
            x = torch.randn(8, 16, generator=g).to(dtype)
            ref = [torch.empty_like(x) for _ in range(2)]
            dist.all_gather(ref, x, group=grid.col_group)
            assert torch.equal(heap.all_gather(x, grid.col_group), torch.cat(ref)), "all_gather after the sparse plans"
            heap.check_symmetric()
        if dtype == torch.float32:                           # two-shot all-reduce of named heap tensors over epoch channels
            n = 1000
            src = heap.empty(n, torch.float32, "grads")
            heap.empty(n, torch.float32, "grads_sum")
            for rep in range(3):
                src.copy_(torch.arange(n, dtype=torch.float32) * (rank + 1) + rep)
                heap.all_reduce_two_shot("grads", "grads_sum", n)
                want = torch.arange(n, dtype=torch.float32) * sum(range(1, world + 1)) + rep * world
                assert torch.equal(heap.view(heap.named["grads_sum"][0], (n,), torch.float32), want), "two-shot all-reduce"
            heap.check_symmetric()
        native.check_status(torch.device("cpu"))
    finally:
        dist.barrier()
        heap.close()


@pytest.mark.parametrize("dtype_name", ["float64", "float32", "bfloat16"])
def test_heap_collectives_match_gloo_on_a_2x2_grid(dtype_name):
    run_dist(_collectives_worker, 4, dtype_name)


def _expiry_worker(rank, world):
    import torch.distributed as dist
    from gt_b200.ops import native
    from gt_b200.parallel.symm_host import HostSymmetricHeap
    heap = HostSymmetricHeap(1 << 20, wait_seconds=0.5)
    ctx = heap.ctx(None)
    dist.barrier()
    if rank != 1:                                            # rank 1 never arrives: the others give up after the limit and say who
        ctx.barrier()
        with pytest.raises(RuntimeError, match="code 101"):
            native.check_status(torch.device("cpu"))
        native.check_status(torch.device("cpu"))             # the word was cleared; the process carries on
    dist.barrier()
    heap.close()


def test_a_silent_rank_expires_the_barrier_with_its_index():
    run_dist(_expiry_worker, 3)
