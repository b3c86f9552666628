"""GEMM microbenchmark: the package's tcgen05 kernels against cuBLAS (torch.matmul) on the Linear shapes of the models
(the GEMM TFLOPS constants of the performance model; counterpart of the GEMM section of the reference's
``gt3d/bench/hw_constants.py``).  One ``GEMM`` line per shape: ms, TFLOP/s and effective GB/s for forward (NT), input
gradient (NT on the transposed weight) and weight gradient (TN), and the cuBLAS time of the same product.

    python -m gt_b200.bench.bench_gemm --rows 169344 --dims 256:768 256:256 256:512 512:256
"""
import argparse
import json

import torch


def timeit(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(iters):
        fn()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=169344)
    ap.add_argument("--dims", nargs="+", default=["256:768", "256:256", "256:512", "512:256", "128:256"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--only", default=None, choices=[None, "nt", "tn", "gather", "scatter"])
    ap.add_argument("--scatter", type=int, default=0, metavar="G",
                    help="also time the reduce-scatter-fused kernel with G owner slots that all live on this GPU")
    ap.add_argument("--gather", type=int, default=0, metavar="G",
                    help="also time the all-gather-fused kernel with G row chunks that all live on this GPU (the kernel's own "
                         "efficiency without the link; multi-GPU timing is in bench_collectives)")
    args = ap.parse_args()
    from ..ops import native
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    m = args.rows
    for spec in args.dims:
        k, n = (int(v) for v in spec.split(":"))
        x = torch.randn(m, k, device=dev).bfloat16()
        w = torch.randn(n, k, device=dev).bfloat16()
        dy = torch.randn(m, n, device=dev).bfloat16()
        flops = 2.0 * m * n * k
        out = dict(M=m, K=k, N=n)
        if args.only in (None, "nt"):
            ms = timeit(lambda: native.gemm_nt(x, w), args.iters, args.warmup)
            ms_ref = timeit(lambda: x @ w.t(), args.iters, args.warmup)
            out.update(nt_ms=ms, nt_tflops=flops / ms / 1e9, nt_gbs=(m * k + m * n + n * k) * 2 / ms / 1e6, cublas_nt_ms=ms_ref)
        if args.only in (None, "tn"):
            ms = timeit(lambda: native.gemm_tn(dy, x), args.iters, args.warmup)
            ms_ref = timeit(lambda: dy.t() @ x, args.iters, args.warmup)
            out.update(tn_ms=ms, tn_tflops=flops / ms / 1e9, cublas_tn_ms=ms_ref)
        if args.gather and k <= 512 and m % args.gather == 0:
            chunk = m // args.gather
            y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            xg = torch.empty_like(x)
            ptrs = [x[i * chunk:].data_ptr() for i in range(args.gather)]
            e = native.ext()

            def fused(copy):
                e.gemm_nt_gather(ptrs, chunk, k, k, w, y, None, 0, 0.0, None, 0, xg if copy else None, native.status(dev), None, None, 0, 0)
            ms = timeit(lambda: fused(False), args.iters, args.warmup)
            ms_c = timeit(lambda: fused(True), args.iters, args.warmup)
            fused(True)
            ok = bool(torch.equal(xg, x)) and float((y.float() - (x @ w.t()).float()).abs().max()) < 0.05 * float((x @ w.t()).float().abs().max())
            out.update(gather_chunks=args.gather, gather_ms=ms, gather_tflops=flops / ms / 1e9, gather_copy_ms=ms_c, gather_ok=ok)
        if args.scatter and m % args.scatter == 0 and n % 8 == 0:
            g_ = args.scatter
            chunk = m // g_
            slots = torch.empty(g_, chunk, n, dtype=torch.bfloat16, device=dev)       # slot p = "owner p's" staging area for this rank
            ptrs = [slots[i].data_ptr() for i in range(g_)]
            e = native.ext()
            ms = timeit(lambda: e.gemm_nt_scatter(x, w, ptrs, chunk, n, native.status(dev)), args.iters, args.warmup)
            ref = (x @ w.t()).view(g_, chunk, n)
            ok = float((slots.float() - ref.float()).abs().max()) < 0.05 * float(ref.float().abs().max())
            out.update(scatter_slots=g_, scatter_ms=ms, scatter_tflops=flops / ms / 1e9, scatter_ok=ok)
        native.check_status(dev)
        print("GEMM " + json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
