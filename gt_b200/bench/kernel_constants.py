"""Fit the linear cost model of the sparse kernels, ``T = c_e E + c_r R + c_c C`` (ns per edge, destination row, source
row), on random blocks, separately for an L2-resident and an HBM-resident gathered operand, and write the slopes as a
JSON overlay for ``gt_b200.perf.grid_select`` (counterpart of the reference's ``gt3d/bench/kernel_constants.py:59-115``
and ``kernel_l2.py``).

    python -m gt_b200.bench.kernel_constants --out gt_b200/perf/b200_constants.json

The L2 regime uses blocks whose K and V rows (2 x C x H x d x 2 bytes) stay below 40 MB, the HBM regime blocks above
400 MB with an L2 flush before every timed launch.  Attention: gated score, clamp-exp norm, bf16 operands, partial
(unnormalised) forward and partial backward (row pass + column pass).  SpMM: weighted CSR times a bf16 matrix.
"""
import argparse
import json
import os

import torch

from ._timing import lstsq_nonneg, time_ms


def random_block(rows, cols, e, types, dev, weight=False, seed=0):
    from ..attention import BlockCSR
    g = torch.Generator().manual_seed(seed)
    ei = torch.stack([torch.randint(0, cols, (e,), generator=g), torch.randint(0, rows, (e,), generator=g)])
    et = torch.randint(0, types, (e,), generator=g)
    w = torch.rand(e, generator=g) if weight else None
    return BlockCSR.from_edges(ei, rows, cols, et, weight=w).to(dev) if weight else BlockCSR.from_edges(ei, rows, cols, et).to(dev)


def attention_points(dev, h, d, shapes, flush, iters):
    from ..attention import backend_cuda as bc
    pts = []
    for rows, cols, e in shapes:
        blk = random_block(rows, cols, e, 3, dev)
        q = torch.randn(rows, h, d, device=dev).bfloat16()
        k, v = (torch.randn(cols, h, d, device=dev).bfloat16() for _ in range(2))
        gate = torch.randn(3, h, d, device=dev)
        kw = dict(score="gated", norm="clampexp")
        acc, l, m = bc.attn_fwd_partial(q, k, v, blk, gate, None, **kw)
        dacc, dl = torch.randn_like(acc), torch.randn_like(l)
        f = time_ms(lambda: bc.attn_fwd_partial(q, k, v, blk, gate, None, **kw), iters, 3, flush=flush)
        b = time_ms(lambda: bc.attn_bwd_partial(q, k, v, blk, gate, None, m, dacc, dl, **kw), iters, 3, flush=flush)
        pts.append((rows, cols, e, f, b))
        print(f"KC attn {'hbm' if flush else 'l2 '} R={rows} C={cols} E={e} fwd {f:.3f} ms bwd {b:.3f} ms", flush=True)
        del blk, q, k, v, acc, dacc
    return pts


def spmm_points(dev, width, shapes, flush, iters):
    from ..ops import native
    pts = []
    for rows, cols, e in shapes:
        blk = random_block(rows, cols, e, 1, dev, weight=True)
        x = torch.randn(cols, width, device=dev).bfloat16()
        t = time_ms(lambda: native.spmm(blk, x), iters, 3, flush=flush)
        pts.append((rows, cols, e, t))
        print(f"KC spmm {'hbm' if flush else 'l2 '} R={rows} C={cols} E={e} {t:.3f} ms", flush=True)
    return pts


def fit(pts, col):
    a = [[e, r, c] for r, c, e, *_ in pts]
    y = [p[col] * 1e6 for p in pts]                             # ns
    return lstsq_nonneg(a, y)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--head_dim", type=int, default=32)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--out", default=None)
    ap.add_argument("--small", action="store_true", help="a tenth of the sizes (smoke test)")
    args = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    s = 10 if args.small else 1
    h, d = args.heads, args.head_dim
    # L2 regime: C <= 32K rows of 512 B for K and V each; vary E, R, C independently
    l2_shapes = [(32768 // s, 32768 // s, 500_000 // s), (32768 // s, 32768 // s, 2_000_000 // s), (262144 // s, 32768 // s, 2_000_000 // s),
                 (262144 // s, 16384 // s, 1_000_000 // s), (65536 // s, 8192 // s, 4_000_000 // s)]
    hbm_shapes = [(524288 // s, 524288 // s, 2_000_000 // s), (524288 // s, 524288 // s, 8_000_000 // s), (1048576 // s, 524288 // s, 4_000_000 // s),
                  (262144 // s, 1048576 // s, 4_000_000 // s), (1048576 // s, 1048576 // s, 12_000_000 // s)]
    a_l2 = attention_points(dev, h, d, l2_shapes, False, args.iters)
    a_hbm = attention_points(dev, h, d, hbm_shapes, True, args.iters)
    s_l2 = spmm_points(dev, h * d, l2_shapes, False, args.iters)
    s_hbm = spmm_points(dev, h * d, hbm_shapes, True, args.iters)
    sp_l2, sp_hbm = fit(s_l2, 3), fit(s_hbm, 3)
    out = dict(attn=dict(fwd=dict(l2=fit(a_l2, 3), hbm=fit(a_hbm, 3)), bwd=dict(l2=fit(a_l2, 4), hbm=fit(a_hbm, 4))),
               attn_ref_width=h * d, spmm=dict(l2=sp_l2[0], hbm=sp_hbm[0], row_ns=0.5 * (sp_l2[1] + sp_hbm[1])),
               _kernel_points=dict(attn_l2=a_l2, attn_hbm=a_hbm, spmm_l2=s_l2, spmm_hbm=s_hbm))
    print("KC " + json.dumps({k: v for k, v in out.items() if not k.startswith("_")}), flush=True)
    if args.out:
        old = {}
        if os.path.exists(args.out):
            with open(args.out) as f:
                old = json.load(f)
        old.update(out)
        with open(args.out, "w") as f:
            json.dump(old, f, indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
