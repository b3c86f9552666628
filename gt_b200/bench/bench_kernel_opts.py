"""Kernel-side options of the attention operator on synthetic blocks, one GPU (counterpart of the reference's
``gt3d/bench/bench_kernel_opts.py``).  For each block shape and each option set: forward and backward (row + column pass) ms.

Blocks (rows x columns, edges) follow the tiles of the benchmark graphs: the whole 169K-node Exphormer graph, its 2 x 4 tile,
a products-like 612K x 612K tile and a dense-ish Reddit-like tile.  Options:

  * operand type: bf16 or fp32 Q / K / V (fp32 takes the register-pipelined kernels, bf16 the cp.async ring kernels);
  * head layout at 256 channels: 8 x 32 (compile-time specialised instance), 4 x 64 and 16 x 16 (generic instance);
  * hub-row segment length (``seg_edges``): rows and columns longer than this are cut into segments merged by a second kernel;
  * ``--no_ring``: re-run the bf16 cases in a child process with ``GT_ATTN_ASYNC=0`` (register-pipelined kernels for bf16).

    python -m gt_b200.bench.bench_kernel_opts [--blocks arxiv tile24] [--no_ring]
"""
import argparse
import json
import os
import subprocess
import sys

import torch

from ._timing import time_ms

BLOCKS = {
    "arxiv": (169344, 169344, 2_500_000),          # one GPU: the whole Exphormer graph without the virtual node
    "tile24": (84672, 42336, 312_000),             # its tile on a 2 x 4 grid
    "products": (612352, 612352, 8_840_000),       # products on a 4 x 4 grid
    "reddit": (14592, 58368, 1_800_000),           # a Reddit tile on 64 ranks: many edges per row
}


def random_block(n_rows, n_cols, edges, types=3, seed=0):
    from ..attention import BlockCSR
    g = torch.Generator().manual_seed(seed)
    ei = torch.stack([torch.randint(0, n_cols, (edges,), generator=g), torch.randint(0, n_rows, (edges,), generator=g)])
    return BlockCSR.from_edges(ei, n_rows, n_cols, torch.randint(0, types, (edges,), generator=g))


def run_case(blk, n_rows, n_cols, h, d, dtype, seg_edges, dev, iters):
    from ..attention import backend_cuda as bc
    torch.manual_seed(0)
    q = torch.randn(n_rows, h, d, device=dev).to(dtype)
    k, v = (torch.randn(n_cols, h, d, device=dev).to(dtype) for _ in range(2))
    gate = torch.randn(3, h, d, device=dev)
    kw = dict(score="gated", norm="clampexp")
    if seg_edges:
        kw["seg_edges"] = seg_edges
    acc, l, m = bc.attn_fwd_partial(q, k, v, blk, gate, None, **kw)
    dacc, dl = torch.randn_like(acc), torch.randn_like(l)
    fwd = time_ms(lambda: bc.attn_fwd_partial(q, k, v, blk, gate, None, **kw), iters=iters, warmup=3, flush=True, dev=dev)
    bwd = time_ms(lambda: bc.attn_bwd_partial(q, k, v, blk, gate, None, m, dacc, dl, **kw), iters=iters, warmup=3, flush=True, dev=dev)
    return fwd, bwd


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--blocks", nargs="+", default=["arxiv", "tile24"], choices=sorted(BLOCKS))
    ap.add_argument("--layouts", nargs="+", default=["8x32", "4x64", "16x16"])
    ap.add_argument("--dtypes", nargs="+", default=["bf16", "fp32"])
    ap.add_argument("--seg_edges", type=int, nargs="+", default=[0], help="0 = the backend's default segment length")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--no_ring", action="store_true", help="also run the bf16 cases with GT_ATTN_ASYNC=0 in a child process")
    args = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    ring = os.environ.get("GT_ATTN_ASYNC", "1") != "0"
    out = []
    for name in args.blocks:
        n_rows, n_cols, edges = BLOCKS[name]
        blk = random_block(n_rows, n_cols, edges).to(dev)
        for lay in args.layouts:
            h, d = (int(x) for x in lay.split("x"))
            for dt in args.dtypes:
                for seg in args.seg_edges:
                    fwd, bwd = run_case(blk, n_rows, n_cols, h, d, torch.bfloat16 if dt == "bf16" else torch.float32, seg, dev, args.iters)
                    row = dict(block=name, rows=n_rows, cols=n_cols, edges=edges, layout=lay, dtype=dt, seg_edges=seg or "default",
                               ring=bool(ring and dt == "bf16"), fwd_ms=fwd, bwd_ms=bwd, fwd_ns_per_edge=fwd * 1e6 / edges,
                               bwd_ns_per_edge=bwd * 1e6 / edges)
                    out.append(row)
                    print("OPTS " + json.dumps(row), flush=True)
    if args.no_ring and ring:
        env = dict(os.environ, GT_ATTN_ASYNC="0")
        cmd = [sys.executable, "-m", "gt_b200.bench.bench_kernel_opts", "--blocks", *args.blocks, "--layouts", *args.layouts,
               "--dtypes", "bf16", "--iters", str(args.iters), "--seg_edges", *[str(s) for s in args.seg_edges]]
        subprocess.run(cmd, env=env, check=True)
    return out


if __name__ == "__main__":
    main()
