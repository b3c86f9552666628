"""One structure-masked sparse attention layer (gated scores, clamp-exp normalisation, edge types) on one GPU: the sm_100a
kernels against other ways of computing the same operator (counterpart of the reference's
``gt3d/bench/bench_kernel_external.py`` and ``bench_sga_kernel.py``).  Forward and forward + backward time, peak extra
memory, and the largest deviation from the edge-list implementation.

  ``edge_list``   gather / scatter over ``[E, H, d]`` messages through autograd (how PyG-style model code computes it),
  ``csr_torch``   this package's CSR backend in plain torch ops with an explicit backward,
  ``sparse_lib``  library pipeline: sampled dense-dense product per head (``torch.sparse.sampled_addmm``), exponentials on
                  the CSR values, sparse-dense product (``torch.sparse.mm``); dot scores only (forward),
  ``dense_sdpa``  dense ``scaled_dot_product_attention`` over the same rows without a mask: the cost floor of every
                  dense or block-dense approach; only up to ``--dense_max`` rows,
  ``cuda``        the package's kernels (``gt_b200.attention.backend_cuda``).

    python -m gt_b200.bench.bench_kernel_external --graph exphormer_arxiv --layouts 8x32 4x32
"""
import argparse
import json

import torch

from ._timing import time_ms


def implementations(blk, ei, et, score):
    from ..attention import backend_cuda as bc, backend_torch as bt
    from ..attention.ref import masked_sparse_attention_ref
    kw = dict(score=score, norm="clampexp")

    def edge_list(q, k, v, gate):
        return masked_sparse_attention_ref(q.float(), k.float(), v.float(), ei, edge_type=et, gate=gate, **kw)

    def csr_torch(q, k, v, gate):
        return bt.masked_sparse_attention_torch(q.float(), k.float(), v.float(), blk, gate=gate, **kw)

    def cuda(q, k, v, gate):
        return bc.masked_sparse_attention_cuda(q, k, v, blk, gate=gate, **kw)

    return dict(edge_list=edge_list, csr_torch=csr_torch, cuda=cuda)


def sparse_lib_forward(q, k, v, blk):
    """Dot-score clamp-exp attention by library sparse kernels, one head at a time (forward only)."""
    n, h, d = q.shape
    crow, col = blk.crow.long(), blk.col.long()
    pattern = torch.sparse_csr_tensor(crow, col, torch.zeros(col.numel(), device=q.device), size=(n, k.shape[0]))
    out = []
    for i in range(h):
        s = torch.sparse.sampled_addmm(pattern, q[:, i].float(), k[:, i].float().t(), beta=0.0, alpha=d ** -0.5)
        p = torch.sparse_csr_tensor(crow, col, s.values().clamp(-5, 5).exp(), size=s.shape)
        num = torch.sparse.mm(p, v[:, i].float())
        den = torch.sparse.mm(p, torch.ones(k.shape[0], 1, device=q.device))
        out.append(num / (den + 1e-6))
    return torch.stack(out, 1)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--graph", default="exphormer_arxiv")
    ap.add_argument("--scale_down", type=int, default=1)
    ap.add_argument("--layouts", nargs="+", default=["8x32"])
    ap.add_argument("--impls", nargs="+", default=["edge_list", "csr_torch", "sparse_lib", "dense_sdpa", "cuda"])
    ap.add_argument("--dense_max", type=int, default=65536)
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args(argv)
    from .bench_attention_single_gpu import build_block
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    blk, n = build_block(argparse.Namespace(random=None, graph=args.graph, scale_down=args.scale_down, no_token=False), dev)
    from ..attention.csr import rows_of_edges
    ei = torch.stack([blk.col.long(), rows_of_edges(blk.crow).long()])
    et = blk.etype.long() if blk.etype is not None else None
    out = []
    for lay in args.layouts:
        h, d = (int(x) for x in lay.split("x"))
        torch.manual_seed(0)
        q, k, v = (torch.randn(n, h, d, device=dev).bfloat16() for _ in range(3))
        gate = torch.randn(3, h, d, device=dev)
        impls = implementations(blk, ei, et, "gated")
        ref = None
        for name in args.impls:
            row = dict(graph=args.graph, nodes=n, edges=blk.num_edges, layout=lay, impl=name)
            try:
                torch.cuda.synchronize()
                torch.cuda.reset_peak_memory_stats(dev)
                base = torch.cuda.memory_allocated(dev)
                if name == "sparse_lib":
                    row["score"] = "dot"
                    row["fwd_ms"] = time_ms(lambda: sparse_lib_forward(q, k, v, blk), iters=args.iters, warmup=3, dev=dev)
                elif name == "dense_sdpa":
                    if n > args.dense_max:
                        row["skipped"] = f"more than {args.dense_max} rows"
                        print("EXTERNAL " + json.dumps(row), flush=True)
                        continue
                    qd, kd, vd = (t.transpose(0, 1).unsqueeze(0).contiguous().requires_grad_() for t in (q, k, v))
                    f = lambda: torch.nn.functional.scaled_dot_product_attention(qd, kd, vd)          # noqa: E731
                    row["fwd_ms"] = time_ms(f, iters=args.iters, warmup=3, dev=dev)
                    row["fwd_bwd_ms"] = time_ms(lambda: f().sum().backward(), iters=args.iters, warmup=3, dev=dev)
                else:
                    fn = impls[name]
                    leaves = [t.clone().requires_grad_() for t in (q, k, v, gate)]
                    with torch.no_grad():
                        o = fn(q, k, v, gate).float()
                    if name == "edge_list":
                        ref = o
                    elif ref is not None:
                        row["max_abs_diff_vs_edge_list"] = float((o - ref).abs().max())
                    row["fwd_ms"] = time_ms(lambda: fn(q, k, v, gate), iters=args.iters, warmup=3, dev=dev)
                    w = torch.randn_like(o)

                    def fb():
                        for t in leaves:
                            t.grad = None
                        (fn(*leaves).float() * w).sum().backward()
                    row["fwd_bwd_ms"] = time_ms(fb, iters=args.iters, warmup=3, dev=dev)
                row["peak_extra_gb"] = (torch.cuda.max_memory_allocated(dev) - base) / 2 ** 30
            except (RuntimeError, NotImplementedError) as e:       # out of memory or an operator the library lacks for this dtype
                row["error"] = str(e).splitlines()[0][:120]
                torch.cuda.empty_cache()
            out.append(row)
            print("EXTERNAL " + json.dumps(row), flush=True)
    return out


if __name__ == "__main__":
    main()
