"""Row-kernel microbenchmark: fused dropout + residual + LayerNorm forward / backward (plain and with the attention
normalisation folded in), SpMM and the column packing kernel on one GPU, with the achieved fraction of a plain copy's
bandwidth (the ``ew_gbs`` constant of the performance model; also the small case used for Nsight Compute captures).

    python -m gt_b200.bench.bench_rowops --rows 169344 --dim 256
"""
import argparse
import json

import torch

from ._timing import time_ms


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", type=int, default=169344)
    ap.add_argument("--dim", type=int, default=256)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--p", type=float, default=0.1)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)
    from ..ops import native
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n, d, h = args.rows, args.dim, args.heads
    y = torch.randn(n, d, device=dev).bfloat16().requires_grad_()
    x = torch.randn(n, d, device=dev).bfloat16().requires_grad_()
    acc = torch.randn(n, d, device=dev).requires_grad_()
    l = (torch.rand(n, h, device=dev) + 0.5).requires_grad_()
    gamma, beta, bias = (torch.ones(d, device=dev).requires_grad_(), torch.zeros(d, device=dev).requires_grad_(),
                         torch.zeros(d, device=dev).requires_grad_())
    go = torch.randn(n, d, device=dev).bfloat16()
    out = {}
    bytes_plain = 3 * n * d * 2
    bytes_acc = n * d * (4 + 2 + 2)

    def fb(fn, tag, nbytes_f, nbytes_b):
        o = fn()
        f = time_ms(fn, args.iters, args.warmup, flush=True)

        def bwd():
            o.backward(go, retain_graph=True)
        b = time_ms(bwd, args.iters, args.warmup, flush=True)
        out[tag] = dict(fwd_ms=f, bwd_ms=b, fwd_gbs=nbytes_f / f / 1e6, bwd_gbs=nbytes_b / b / 1e6)
    fb(lambda: native.layer_norm(y, x, bias, gamma, beta, 1e-5, args.p), "ln", bytes_plain, 5 * n * d * 2)
    fb(lambda: native.layer_norm(acc, x, None, gamma, beta, 1e-5, args.p, l), "ln_acc", bytes_acc, n * d * (2 + 4 + 2 + 4 + 2))
    parts = [acc.detach(), l.detach().repeat(1, 1), x.detach()]
    pk = time_ms(lambda: native.pack_columns(parts, torch.bfloat16), args.iters, args.warmup, flush=True)
    out["pack"] = dict(ms=pk, gbs=(n * d * 4 + n * h * 4 + n * d * 2 + n * (2 * d + h) * 2) / pk / 1e6)
    native.check_status(dev)
    print("ROWOPS " + json.dumps(dict(rows=n, dim=d, **out)), flush=True)


if __name__ == "__main__":
    main()
