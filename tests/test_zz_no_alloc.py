"""The allocation-free aggregation entry point ``gt_spmm_csr_noalloc`` (declared in ``gt_b200/csrc/noalloc.h``).

Some hosts of the library cannot allocate device memory while they run (all memory handed out at start-up, a fixed part of the
device memory next to other components, or a plain C embedder without a tensor framework).  For them the library keeps the split-row
scratch of the sparse aggregation in a built-in device array.  The test calls the exported C symbol through ``ctypes`` with
raw device pointers, twice in a row (the second call finds the previous call's data in the shared scratch), and compares
with the regular entry point ``gt_b200.ops.native.spmm``; it also checks that a request beyond the built-in capacity is
refused with a message instead of being launched.  The file name sorts last so that a run that stops at the first failure
has already executed every other test.
"""
import ctypes
import glob
import os

import pytest
import torch

from helpers import random_graph

pytestmark = pytest.mark.gpu


def _lib():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cands = sorted(glob.glob(os.path.join(root, "gt_b200", "_ext", "gt_b200_native*.so")))
    assert cands, "native extension not built"
    import torch  # noqa: F401  (libtorch must be loaded before the extension's shared object)
    lib = ctypes.CDLL(cands[-1])
    p, i = ctypes.c_void_p, ctypes.c_int
    lib.gt_spmm_csr_noalloc.argtypes = [i, p, p, p, p, p, i, i, p, p, p, p, i, p, p, i, i, p]
    lib.gt_spmm_csr_noalloc.restype = i
    lib.gt_noalloc_last_error.restype = ctypes.c_char_p
    lib.gt_noalloc_scratch_floats.restype = ctypes.c_size_t
    return lib


def _call(lib, blk, plan, x, out, n_slots=None, use_weight=True):
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())          # noqa: E731
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    dtype = 1 if x.dtype == torch.bfloat16 else 0
    w = ptr(blk.weight) if use_weight else ctypes.c_void_p(0)
    return lib.gt_spmm_csr_noalloc(dtype, ptr(blk.crow), ptr(blk.col), w, ptr(x), ptr(out), blk.n_rows, x.shape[1],
                                   ptr(plan.seg_row), ptr(plan.seg_beg), ptr(plan.seg_end), ptr(plan.seg_slot), plan.num_segments,
                                   ptr(plan.split_rows), ptr(plan.split_ptr), int(plan.split_rows.numel()),
                                   plan.num_slots if n_slots is None else n_slots, stream)


@pytest.mark.parametrize("dtype,d,weighted", [(torch.float32, 128, True), (torch.bfloat16, 256, True), (torch.bfloat16, 512, True),
                                              (torch.float32, 1024, True), (torch.bfloat16, 256, False)])
def test_noalloc_matches_regular_entry_point_twice(dtype, d, weighted):
    from gt_b200.attention import BlockCSR
    from gt_b200.ops import native
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    lib = _lib()
    n = 1500
    ei, _ = random_graph(n, 5, seed=11)                      # node 1 is a hub row with n in-edges -> split rows
    # w = NULL means "all weights one": the regular entry point is then given a block whose weights are ones
    blk = BlockCSR.from_edges(ei, n, n, weight=torch.rand(ei.shape[1]) if weighted else torch.ones(ei.shape[1])).to(dev)
    plan = blk.row_plan(64)
    assert plan.num_slots > 0 and plan.num_slots * d <= lib.gt_noalloc_scratch_floats()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for trial in range(2):
        x = torch.randn(n, d, device=dev, generator=torch.Generator(device=dev).manual_seed(trial)).to(dtype)
        ref = native.spmm(blk, x)                            # regular entry point (scratch from the caching allocator)
        out = torch.full_like(ref, float("nan"))
        rc = _call(lib, blk, plan, x, out, use_weight=weighted)
        torch.cuda.synchronize()
        assert rc == 0, lib.gt_noalloc_last_error().decode()
        err = (out.float() - ref.float()).abs().max().item() / max(ref.float().abs().max().item(), 1e-6)
        assert err < tol, (trial, err)


def test_noalloc_empty_plan_zero_fills():
    from gt_b200.attention import BlockCSR
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    lib = _lib()
    ei, _ = random_graph(64, 3, seed=5)
    blk = BlockCSR.from_edges(ei, 64, 64, weight=torch.rand(ei.shape[1])).to(dev)
    plan = blk.row_plan(16)
    x = torch.randn(64, 32, device=dev)
    out = torch.full((64, 32), float("nan"), device=dev)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())          # noqa: E731
    rc = lib.gt_spmm_csr_noalloc(0, ptr(blk.crow), ptr(blk.col), ptr(blk.weight), ptr(x), ptr(out), 64, 32, ptr(plan.seg_row),
                                 ptr(plan.seg_beg), ptr(plan.seg_end), ptr(plan.seg_slot), 0, ptr(plan.split_rows), ptr(plan.split_ptr),
                                 0, 0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert rc == 0 and out.abs().max().item() == 0


def test_noalloc_rejects_oversized_scratch():
    from gt_b200.attention import BlockCSR
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    lib = _lib()
    ei, _ = random_graph(300, 4, seed=2)
    blk = BlockCSR.from_edges(ei, 300, 300, weight=torch.rand(ei.shape[1])).to(dev)
    plan = blk.row_plan(16)
    x = torch.randn(300, 64, device=dev)
    out = torch.zeros(300, 64, device=dev)
    too_many = lib.gt_noalloc_scratch_floats() // 64 + 1
    rc = _call(lib, blk, plan, x, out, n_slots=too_many)
    assert rc == 1 and b"capacity" in lib.gt_noalloc_last_error()
    assert out.abs().max().item() == 0                       # nothing was launched
