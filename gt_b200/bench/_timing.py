"""Timing helpers shared by the benchmarks: CUDA events on the launching stream after warm-up, an L2 flush between timed
iterations, the maximum over ranks for anything multi-rank."""
import torch
import torch.distributed as dist

_FLUSH = {}


def flush_l2(dev):
    """Overwrite a buffer larger than the 126 MB L2 so the next kernel starts from HBM."""
    buf = _FLUSH.get(dev)
    if buf is None:
        buf = _FLUSH[dev] = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    buf.zero_()


def time_ms(fn, iters=10, warmup=3, flush=False, dev=None, max_over_ranks=False):
    """Mean device time of ``fn`` in ms.  With ``flush`` every iteration is timed on its own after an L2 flush."""
    dev = dev or torch.device("cuda", torch.cuda.current_device())
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(dev)
    if flush:
        tot = 0.0
        for _ in range(iters):
            flush_l2(dev)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            tot += a.elapsed_time(b)
        ms = tot / iters
    else:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        b.synchronize()
        ms = a.elapsed_time(b) / iters
    if max_over_ranks and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def lstsq_nonneg(rows, y):
    """Least-squares slopes of ``y = rows @ c`` with negative slopes clamped to zero and the rest re-fitted."""
    a = torch.tensor(rows, dtype=torch.float64)
    b = torch.tensor(y, dtype=torch.float64).view(-1, 1)
    active = list(range(a.shape[1]))
    c = torch.zeros(a.shape[1], dtype=torch.float64)
    while active:
        sol = torch.linalg.lstsq(a[:, active], b).solution.view(-1)
        if (sol >= 0).all():
            for i, j in enumerate(active):
                c[j] = sol[i]
            break
        active.pop(int(sol.argmin()))
    return [float(v) for v in c]
