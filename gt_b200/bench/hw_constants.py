"""Measure the hardware constants of the performance model on this machine and write them as a JSON overlay for
``gt_b200.perf.grid_select.load_constants`` (counterpart of the reference's ``gt3d/bench/hw_constants.py``).

    python -m gt_b200.bench.hw_constants --out gt_b200/perf/b200_constants.json                (1 GPU: memory, GEMM, kernels gap)
    torchrun --nproc-per-node 8 -m gt_b200.bench.hw_constants --only coll --out coll8.json      (collectives, NCCL and peer-memory)

Sections (``--only`` takes a comma list): ``hbm`` STREAM-style copy; ``gap`` device gap between dependent kernels in a
replayed CUDA graph; ``ew`` achieved bandwidth of the fused dropout + residual + LayerNorm kernels; ``gemm`` TFLOP/s of
the tcgen05 GEMMs (forward, input gradient, weight gradient) per hidden size; ``coll`` latency and large-message rate of
all-gather / reduce-scatter / all-to-all / all-reduce over the world group, for NCCL and for the symmetric-heap kernels.
Every number is device time (CUDA events, max over ranks); inputs are larger than L2 or L2 is flushed between iterations.
"""
import argparse
import json
import os

import torch
import torch.distributed as dist

from ._timing import time_ms


def measure_hbm(dev):
    n = 1 << 30
    a, b = torch.empty(n, dtype=torch.uint8, device=dev), torch.empty(n, dtype=torch.uint8, device=dev)
    ms = time_ms(lambda: b.copy_(a), 10, 3)
    return 2 * n / ms / 1e6


def measure_gap(dev):
    x = torch.zeros(1024, device=dev)
    n = 200
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        x.add_(1.0)
        torch.cuda.synchronize()
        with torch.cuda.graph(g):
            for _ in range(n):
                x.add_(1.0)
    torch.cuda.synchronize()
    return time_ms(g.replay, 10, 3) / n * 1e3


def measure_ew(dev, rows=1 << 20, d=256):
    from ..ops import native
    y, x = (torch.randn(rows, d, device=dev).bfloat16() for _ in range(2))
    gamma, beta, bias = torch.ones(d, device=dev), torch.zeros(d, device=dev), torch.zeros(d, device=dev)
    ms = time_ms(lambda: native.layer_norm(y, x, bias, gamma, beta, 1e-5, 0.1), 10, 3)
    return 3 * rows * d * 2 / ms / 1e6                          # reads y and x, writes the result


def measure_gemm(dev, rows=169344, dims=(128, 256, 512)):
    from ..ops import native
    out = {}
    for d in dims:
        x = torch.randn(rows, d, device=dev).bfloat16()
        w = torch.randn(3 * d, d, device=dev).bfloat16()
        wt = w.t().contiguous()
        dy = torch.randn(rows, 3 * d, device=dev).bfloat16()
        fl = 2.0 * rows * d * 3 * d
        f = time_ms(lambda: native.gemm_nt(x, w), 10, 3, flush=True)
        gi = time_ms(lambda: native.gemm_nt(dy, wt), 10, 3, flush=True)
        gw = time_ms(lambda: native.gemm_tn(dy, x), 10, 3, flush=True)
        out[str(d)] = [fl / f / 1e9, fl / gi / 1e9, fl / gw / 1e9]
    return out


def measure_coll(dev, sizes_mb=(0.25, 1, 4, 16, 64, 256), heap_mb=1280):
    """Per kind: (latency us, GB/s per rank at the largest size) fitted from a size sweep; ``p2p`` from the heap kernels."""
    world, rank = dist.get_world_size(), dist.get_rank()
    heap = None
    try:
        from ..parallel.symm import SymmetricHeap
        heap = SymmetricHeap(dev, heap_mb << 20)
    except Exception as exc:                                    # peer access unavailable: NCCL numbers only
        if rank == 0:
            print(f"HW coll: symmetric heap unavailable ({exc})", flush=True)
    table, curves = {}, {}
    for kind in ("ag", "rs", "a2a", "ar", "p2p"):
        pts = []
        for mb in sizes_mb:
            per = int(mb * 2 ** 20) // 2 // world * world          # bf16 elements per rank
            if per == 0:
                continue
            small, big = torch.randn(per, device=dev).bfloat16(), torch.empty(per * world, dtype=torch.bfloat16, device=dev)
            if kind == "ag":
                fn, payload = (lambda: dist.all_gather_into_tensor(big, small)), per * 2 * (world - 1)
            elif kind == "rs":
                fn, payload = (lambda: dist.reduce_scatter_tensor(small, big)), per * 2 * (world - 1)
            elif kind == "a2a":
                o = torch.empty_like(big)
                fn, payload = (lambda: dist.all_to_all_single(o, big)), per * 2 * (world - 1)
            elif kind == "ar":
                fn, payload = (lambda: dist.all_reduce(big)), 2 * per * world * 2 * (world - 1) / world
            else:
                if heap is None or per * 2 > (heap_mb << 20) // 2:
                    continue
                def fn(small=small):
                    heap.begin_step()                               # resets the call-site sequence: the staging buffer is reused
                    heap.all_gather(small, None)
                payload = per * 2 * (world - 1)
            ms = time_ms(fn, 10, 3, max_over_ranks=True)
            pts.append((payload, ms))
        if not pts:
            continue
        curves[kind] = [(p / 2 ** 20, ms) for p, ms in pts]
        alpha_us = pts[0][1] * 1e3
        p_big, ms_big = pts[-1]
        rate = p_big / max(ms_big - pts[0][1], 1e-6) / 1e6
        table[kind] = [alpha_us, rate]
    return table, curves


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--only", default="hbm,gap,ew,gemm,coll")
    ap.add_argument("--out", default=None)
    ap.add_argument("--rows", type=int, default=169344)
    args = ap.parse_args(argv)
    only = set(args.only.split(","))
    multi = "RANK" in os.environ
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if multi:
        dist.init_process_group("nccl", device_id=dev)
    rank = dist.get_rank() if multi else 0
    out = {"_device": torch.cuda.get_device_name(dev), "_world": dist.get_world_size() if multi else 1}
    if "hbm" in only:
        out["hbm_gbs"] = measure_hbm(dev)
    if "gap" in only:
        out["kernel_gap_us"] = measure_gap(dev)
    if "ew" in only:
        out["ew_gbs"] = measure_ew(dev)
    if "gemm" in only:
        out["gemm_tflops"] = measure_gemm(dev, args.rows)
    if "coll" in only and multi and dist.get_world_size() > 1:
        out["coll"], out["_coll_curves_mb_ms"] = measure_coll(dev)
    if rank == 0:
        print("HW " + json.dumps(out), flush=True)
        if args.out:
            old = {}
            if os.path.exists(args.out):
                with open(args.out) as f:
                    old = json.load(f)
            old.update(out)
            with open(args.out, "w") as f:
                json.dump(old, f, indent=1, sort_keys=True)
    if multi:
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)


if __name__ == "__main__":
    main()
