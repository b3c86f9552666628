"""Step-level observability: per-kernel device-time totals and a census of the tensors autograd keeps for backward.

``kernel_profile`` is the ``--profile`` switch of the trainer (reference: ``_profile_totals``,
``gt3d/gt3d/train/train_dist.py:29-75``): device time per kernel name for one epoch, grouped into the categories the
performance model uses (attention, SpMM, GEMM, norm / elementwise, collectives, optimizer, other).  With the environment
variable ``GT_PROF_TRACE=<prefix>`` it also writes the chrome trace of the epoch to ``<prefix>_rank<r>.json``.
``saved_tensor_census`` is ``--saved_census`` (reference ``_saved_census``, ``train_dist.py:78-118``): every tensor saved
for backward during one forward, deduplicated by storage, in units of one fp32 owned chunk ``[N/P, d]``; the memory
model's per-layer multipliers are read off this table.
"""
import collections
import contextlib
import os

import torch
import torch.distributed as dist

CATEGORIES = (
    ("attention", ("attn_fwd", "attn_bwd", "attn_", "reduce_partials", "combine_slots")),
    ("spmm", ("spmm", "csrmm", "cusparse")),
    ("gemm", ("gemm", "cutlass", "nvjet", "cublas", "tcgen05")),
    ("collective", ("nccl", "pull_", "group_barrier", "all_gather", "reduce_scatter")),
    ("norm/elementwise", ("layer_norm", "ln_", "dropout", "elementwise", "vectorized", "gated_residual", "cross_entropy", "ce_")),
    ("optimizer", ("adamw", "multi_tensor", "grad_norm")),
)


def categorise(name):
    low = name.lower()
    for cat, keys in CATEGORIES:
        if any(k in low for k in keys):
            return cat
    return "other"


@contextlib.contextmanager
def kernel_profile(rank=0, world=1, top=25, file=None):
    from torch.profiler import ProfilerActivity, profile
    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
    with profile(activities=acts) as prof:
        yield
        if torch.cuda.is_available():
            torch.cuda.synchronize()
    trace = os.environ.get("GT_PROF_TRACE")
    if trace:                                       # chrome trace per rank, for gt_b200.bench.analyze_trace
        prof.export_chrome_trace(f"{trace}_rank{rank}.json")
    per_kernel, per_cat = collections.Counter(), collections.Counter()
    calls = collections.Counter()
    for ev in prof.events():
        if getattr(ev, "device_type", None) is not None and "cuda" in str(ev.device_type).lower():
            us = getattr(ev, "device_time", 0.0) or getattr(ev, "cuda_time", 0.0) or 0.0
            per_kernel[ev.name] += us
            calls[ev.name] += 1
            per_cat[categorise(ev.name)] += us
    if rank == 0:
        total = sum(per_kernel.values()) or 1.0
        print(f"[profile] device time of one epoch on rank 0: {total / 1e3:.2f} ms in {sum(calls.values())} kernels", file=file)
        for cat, us in per_cat.most_common():
            print(f"[profile]   {cat:18s} {us / 1e3:9.3f} ms  {100 * us / total:5.1f} %", file=file)
        for name, us in per_kernel.most_common(top):
            print(f"[profile]   {us / 1e3:9.3f} ms x{calls[name]:<5d} {name[:110]}", file=file)


@contextlib.contextmanager
def saved_tensor_census(grid=None, rank=0, hidden=None, file=None):
    seen, rows = set(), collections.Counter()
    count = collections.Counter()

    def pack(t):
        if isinstance(t, torch.Tensor) and t.numel() > 0:
            st = t.untyped_storage()
            key = (st.data_ptr(), t.storage_offset(), tuple(t.shape), t.dtype)
            if key not in seen and not isinstance(t, torch.nn.Parameter):
                seen.add(key)
                label = (tuple(t.shape), str(t.dtype).split(".")[-1])
                rows[label] += t.numel() * t.element_size()
                count[label] += 1
        return t

    with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
        yield rows
    if rank == 0:
        total = sum(rows.values())
        unit = None
        if grid is not None and hidden:
            unit = grid.chunk * hidden * 4
        print(f"[saved_census] {len(rows)} distinct shapes, {total / 2 ** 20:.1f} MiB saved for backward"
              + (f" = {total / unit:.1f} owned fp32 chunks [N/P, d]" if unit else ""), file=file)
        for label, nb in rows.most_common(30):
            print(f"[saved_census]   {nb / 2 ** 20:10.2f} MiB  x{count[label]:<3d} {label[1]:9s} {label[0]}", file=file)


def structure_bytes(*objs):
    """Bytes of the integer / weight tensors held by graph-structure objects (CSR, CSC, plans), deduplicated by storage."""
    seen, total = set(), 0

    def walk(o):
        nonlocal total
        if isinstance(o, torch.Tensor):
            k = o.untyped_storage().data_ptr()
            if k not in seen:
                seen.add(k)
                total += o.untyped_storage().nbytes()
        elif isinstance(o, dict):
            for v in o.values():
                walk(v)
        elif isinstance(o, (list, tuple)):
            for v in o:
                walk(v)
        elif hasattr(o, "__dict__") and not isinstance(o, torch.nn.Module):
            walk(vars(o))
    for o in objs:
        walk(o)
    return total
