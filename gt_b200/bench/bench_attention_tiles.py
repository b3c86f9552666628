"""Tensor-core tile attention against the gather kernels on masks with dense 128 x 128 tiles.

    python -m gt_b200.bench.bench_attention_tiles --nodes 131072 --heads 16 --density 0.03 0.1 0.3

Builds a clustered mask (communities of ``--community`` nodes whose internal mask holds the given fraction of its entries,
plus ``--background`` random edges per row), and times the forward on (a) the gather kernels alone and (b) the density dispatch
(dense tiles on ``attn_tile_fwd_kernel``, residual on the gather kernels).  CUDA events, L2 flushed between timed launches.
One ``TILE`` line per density: edges, tiles, ms of both paths, and the dense-tile product rate of the tile kernel
(4 * 128 * 128 * 32 FLOP per tile and head for ``Q K^T`` and ``P V``).  ``--only tile`` runs path (b) alone (profiler captures).
"""
import argparse
import json

import torch


def clustered_block(n, density, background, types, dev, seed=0, community=128):
    from ..attention import BlockCSR
    g = torch.Generator(device=dev).manual_seed(seed)
    n_cl = n // community
    on = torch.rand(n_cl, community, community, device=dev, generator=g) < density
    c, r, s = on.nonzero(as_tuple=True)
    dst, src = c * community + r, c * community + s
    if background:
        bd = torch.arange(n, device=dev).repeat_interleave(background)
        bs = torch.randint(0, n, (bd.numel(),), device=dev, generator=g)
        dst, src = torch.cat([dst, bd]), torch.cat([src, bs])
    key = torch.unique(dst * n + src)
    dst, src = key // n, key % n
    et = torch.randint(0, types, (key.numel(),), device=dev, generator=g)
    return BlockCSR.from_edges(torch.stack([src, dst]), n, n, et)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--nodes", type=int, default=131072)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--density", type=float, nargs="+", default=[0.03, 0.1, 0.3])
    ap.add_argument("--background", type=int, default=4)
    ap.add_argument("--community", type=int, default=128, help="nodes per community: community / 128 dense tiles per row block")
    ap.add_argument("--types", type=int, default=3)
    ap.add_argument("--score", default="biased", choices=["dot", "biased"])
    ap.add_argument("--norm", default="softmax", choices=["softmax", "clampexp"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--only", default="both", choices=["both", "tile"])
    args = ap.parse_args()
    from ..attention import backend_cuda as bc
    from ..attention import tiles as tl
    from ..ops import native
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n, h, d = args.nodes // 128 * 128, args.heads, 32
    torch.manual_seed(0)
    q, k, v = (torch.randn(n, h, d, device=dev).bfloat16() for _ in range(3))
    bias = torch.randn(args.types, h, device=dev) if args.score == "biased" else None
    kw = dict(score=args.score, norm=args.norm)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timeit(fn):
        for _ in range(args.warmup):
            fn()
        ms = 0.0
        for _ in range(args.iters):
            flush.zero_()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            fn()
            t1.record()
            torch.cuda.synchronize()
            ms += t0.elapsed_time(t1)
        return ms / args.iters

    for dens in args.density:
        blk = clustered_block(n, dens, args.background, args.types, dev, community=args.community)
        plan = tl.build_tile_plan(blk, min_share=0.0)
        out = dict(nodes=n, heads=h, density=dens, community=args.community, edges=blk.num_edges, tiles=plan.num_tiles if plan else 0,
                   tiled_edges=plan.num_tiled_edges if plan else 0)
        if args.only == "both":
            blk._cache["tile_plan"] = None
            out["gather_ms"] = round(timeit(lambda: bc.attn_fwd_partial(q, k, v, blk, None, bias, **kw)), 4)
            ref = bc.attn_fwd_partial(q, k, v, blk, None, bias, **kw)
        if plan is not None:
            blk._cache["tile_plan"] = plan
            out["dispatch_ms"] = round(timeit(lambda: bc.attn_fwd_partial(q, k, v, blk, None, bias, **kw)), 4)
            acc, l, m = (torch.zeros(n, h, d, device=dev), torch.zeros(n, h, device=dev), torch.zeros(n, h, device=dev))
            out["tile_kernel_ms"] = round(timeit(lambda: bc.attn_tile_accumulate(q, k, v, plan, bias, acc, l, m, **kw)), 4)
            out["tile_tflops"] = round(plan.num_tiles * h * 4 * 128 * 128 * 32 / out["tile_kernel_ms"] / 1e9, 1)
            if args.only == "both":
                got = bc.attn_fwd_partial(q, k, v, blk, None, bias, **kw)
                o_ref, o_got = bc.normalize(ref[0], ref[1], args.norm), bc.normalize(got[0], got[1], args.norm)
                out["max_abs_diff"] = round((o_ref - o_got).abs().max().item(), 5)
        native.check_status(dev)
        print("TILE " + json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
