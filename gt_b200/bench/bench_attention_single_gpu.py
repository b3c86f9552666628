"""Single-GPU attention operator benchmark: forward, backward row pass + column pass of the sm_100a kernels on a named
synthetic graph or a random block (the measurement behind the ``attn`` constants of the performance model; counterpart of
the reference's ``gt3d/bench/bench_attention_single_gpu.py`` / ``hw_constants.py`` attention section).

    python -m gt_b200.bench.bench_attention_single_gpu --graph exphormer_arxiv --heads 8 --head_dim 32 --dtype bf16
    python -m gt_b200.bench.bench_attention_single_gpu --random 612352 8840000 --heads 4 --head_dim 32

Prints one ``ATTN`` line: ms per pass, ns per edge and "model bytes" GB/s, where the model traffic of a pass is what an
ideal kernel without cache reuse would move: per edge two gathered feature rows (K and V, or Q and dAcc), per row / column
its own operands and results.  Timed with CUDA events after warm-up; the gathered operands (2 x N x H x d elements) are larger
than L2 for the named graphs.
"""
import argparse
import json

import torch


def build_block(args, dev):
    from ..attention import BlockCSR
    if args.random:
        n, e = args.random
        g = torch.Generator().manual_seed(0)
        ei = torch.randint(0, n, (2, e), generator=g)
        et = torch.randint(0, args.types, (e,), generator=g)
        return BlockCSR.from_edges(ei, n, n, et).to(dev), n
    from ..data.expander import keyed_expander_edges
    from ..data.synthetic import virtual_node_edges, workload_graph
    from ..models.exphormer_ref import ExphormerRef
    wl = workload_graph(args.graph, seed=0, scale_down=args.scale_down)
    n = wl["n"]
    exp = keyed_expander_edges(n, 4, seed=0)
    tok = virtual_node_edges(n)[0] if not args.no_token else None
    ei, et = ExphormerRef.build_attention_edges(wl["edge_index"], exp, tok)
    n_tot = n + (0 if args.no_token else 1)
    return BlockCSR.from_edges(ei, n_tot, n_tot, et).to(dev), n_tot


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--graph", default="exphormer_arxiv")
    ap.add_argument("--random", type=int, nargs=2, default=None, metavar=("N", "E"))
    ap.add_argument("--scale_down", type=int, default=1)
    ap.add_argument("--no_token", action="store_true")
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--head_dim", type=int, default=32)
    ap.add_argument("--types", type=int, default=3)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--score", default="gated")
    ap.add_argument("--norm", default="clampexp")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seg_edges", type=int, default=None)
    args = ap.parse_args()
    from ..attention import backend_cuda as bc
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    blk, n = build_block(args, dev)
    h, d = args.heads, args.head_dim
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    torch.manual_seed(0)
    q, k, v = (torch.randn(n, h, d, device=dev).to(dt) for _ in range(3))
    gate = torch.randn(args.types, h, d, device=dev) if args.score == "gated" else None
    bias = torch.randn(args.types, h, device=dev) if args.score == "biased" else None
    kw = dict(score=args.score, norm=args.norm)
    if args.seg_edges:
        kw["seg_edges"] = args.seg_edges
    acc, l, m = bc.attn_fwd_partial(q, k, v, blk, gate, bias, **kw)
    dacc, dl = torch.randn_like(acc), torch.randn_like(l)

    def timeit(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.iters):
            fn()
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / args.iters

    ms_f = timeit(lambda: bc.attn_fwd_partial(q, k, v, blk, gate, bias, **kw))
    ms_b = timeit(lambda: bc.attn_bwd_partial(q, k, v, blk, gate, bias, m, dacc, dl, **kw))
    e = blk.num_edges
    es = q.element_size()
    hd = h * d
    fwd_bytes = e * (2 * hd * es + 8) + n * (hd * es + hd * 4 + 8 * h)
    bwd_bytes = 2 * e * (2 * hd * es + 8) + n * (6 * hd * es + 16 * h)
    out = dict(nodes=n, edges=e, heads=h, head_dim=d, dtype=args.dtype, score=args.score, norm=args.norm,
               fwd_ms=ms_f, bwd_ms=ms_b, fwd_ns_per_edge=ms_f * 1e6 / e, bwd_ns_per_edge=ms_b * 1e6 / e,
               fwd_model_gbs=fwd_bytes / ms_f / 1e6, bwd_model_gbs=bwd_bytes / ms_b / 1e6)
    print("ATTN " + json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
