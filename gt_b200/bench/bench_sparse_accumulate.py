"""Which kernel should sum the rows that a sparse reduce-scatter receives (``SparseRowPlan._accumulate``)?

``[n_send, F]`` received rows -> ``[n_rows, F]`` sums over the holders of every owned row, with a static structure (the owned
row of every received row, grouped by sender).  Candidates, timed on one device:

  segment_sum   this package's deterministic segmented sum (the SpMM kernel with unit weights over the stored order)
  index_add     ``index_add_`` into an fp32 buffer (atomics: order, and so the last bits, vary from run to run)
  sort+segment  permutation + ``torch.segment_reduce`` on fp32 copies
  index_copy    one holder per row only: a plain permutation

    python -m gt_b200.bench.bench_sparse_accumulate [--cases ROWS:HOLDERS:WIDTH ...]

Counterpart of the reference's ``gt3d/bench/bench_sparse_accumulate.py`` (which compares ``torch_scatter.segment_csr``,
``index_add_`` and a cuSPARSE product).  Prints one ``ACC`` line per case; returns the list of result dicts.
"""
import argparse
import json
import time

import torch

DEFAULT_CASES = ["612352:1:264", "612352:2:256", "100000:38:256"]


def _time(fn, dev, iters):
    if dev.type == "cuda":
        from ._timing import time_ms
        return time_ms(fn, iters, 3, flush=True, dev=dev)
    fn()
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    return (time.perf_counter() - t0) / iters * 1e3


def run_case(n_rows, holders, width, dev, dtype, iters=10):
    """Every one of ``holders`` senders holds every row: the worst case for a given share."""
    n_send = n_rows * holders
    send_idx = torch.arange(n_rows, device=dev).repeat(holders)
    recv = torch.randn(n_send, width, device=dev).to(dtype)
    perm = torch.argsort(send_idx, stable=True)
    ptr = torch.zeros(n_rows + 1, dtype=torch.long, device=dev)
    ptr[1:] = torch.cumsum(torch.bincount(send_idx, minlength=n_rows), 0)
    lengths = ptr[1:] - ptr[:-1]
    res = dict(rows=n_rows, holders=holders, width=width, dtype=str(dtype).split(".")[-1], mb=round(recv.numel() * recv.element_size() / 1e6, 1))
    ref = torch.zeros(n_rows, width, dtype=torch.float32, device=dev).index_add_(0, send_idx, recv.float())

    def check(out, name):
        err = (out.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
        assert err < (2e-2 if dtype == torch.bfloat16 else 1e-5), (name, err)

    if dev.type == "cuda":
        from ..ops import native
        p32, q32 = perm.to(torch.int32).contiguous(), ptr.to(torch.int32).contiguous()
        out = torch.empty(n_rows, width, dtype=dtype, device=dev)
        check(native.segment_sum_rows(recv, p32, q32, out), "segment_sum")
        res["segment_sum_ms"] = round(_time(lambda: native.segment_sum_rows(recv, p32, q32, out), dev, iters), 4)
    f = lambda: torch.zeros(n_rows, width, dtype=torch.float32, device=dev).index_add_(0, send_idx, recv.float()).to(dtype)   # noqa: E731
    check(f(), "index_add")
    res["index_add_ms"] = round(_time(f, dev, iters), 4)
    g = lambda: torch.segment_reduce(recv.index_select(0, perm).float(), "sum", lengths=lengths).to(dtype)                    # noqa: E731
    check(g(), "sort+segment")
    res["sort_segment_ms"] = round(_time(g, dev, iters), 4)
    if holders == 1:
        h = lambda: torch.empty(n_rows, width, dtype=dtype, device=dev).index_copy_(0, send_idx, recv)                        # noqa: E731
        check(h(), "index_copy")
        res["index_copy_ms"] = round(_time(h, dev, iters), 4)
    return res


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--cases", nargs="+", default=DEFAULT_CASES, metavar="ROWS:HOLDERS:WIDTH")
    ap.add_argument("--dtype", default=None, choices=["bf16", "fp32"])
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args(argv)
    dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    dtype = {"bf16": torch.bfloat16, "fp32": torch.float32, None: torch.bfloat16 if dev.type == "cuda" else torch.float32}[args.dtype]
    out = []
    for case in args.cases:
        n_rows, holders, width = (int(v) for v in case.split(":"))
        out.append(run_case(n_rows, holders, width, dev, dtype, args.iters))
        print("ACC " + json.dumps(out[-1]), flush=True)
    return out


if __name__ == "__main__":
    main()
