"""Planner: what the performance and memory model (:mod:`gt_b200.perf.grid_select`) predicts for a graph on a number of B200s.

Prints, for every layout of the world size (fused 2D grids, head-axis grids, the streamed layer with the smallest number of
column sub-blocks that fits, the ring), the predicted time of one training step and the predicted peak memory per GPU, whether it
fits, and the ``train_dist`` flags that select it.  The trainer's ``--grid_auto`` / ``--head_auto`` / ``--auto_ckpt`` take the same
decisions at run time; this is the table behind them, for sizing a run before GPUs are booked.

    python -m gt_b200.perf.plan --nodes 169344 --edges 2332486 --features 128 --gpus 8 --token
    python -m gt_b200.perf.plan --nodes 67108864 --edges 1073741824 --features 128 --layers 2 --gpus 8
    python -m gt_b200.perf.plan --workload exphormer_arxiv --gpus 4 --json

The time model is calibrated on the fused Exphormer layer of the 169K-node benchmark graph (constants in
``perf/b200_constants.json``); the streamed and ring predictions are extrapolations that were compared with two measured runs
only (within 25-40 %), the memory predictions of the streamed layer with two (within 6 %).
"""
import argparse
import json

from . import grid_select as gs

WORKLOADS = {
    # name: nodes, directed graph edges, input features, classes, expander degree, global token
    "exphormer_arxiv": dict(nodes=169_344, edges=2_332_486, features=128, classes=40, exp_deg=4, token=True),
    "unimp_products": dict(nodes=2_449_029, edges=123_718_280 // 3, features=100, classes=47, exp_deg=0, token=False),
    "exphormer_rmat26": dict(nodes=1 << 26, edges=1 << 30, features=128, classes=172, exp_deg=4, token=False),
}


def layouts(world, g, m, capacity_gb=gs.CAPACITY_GB, headroom=gs.HEADROOM):
    """Rows ``dict(family, grid, n_sub, ms, gb, fits, flags)`` for every layout of ``world`` GPUs, fastest first."""
    rows = []
    limit = capacity_gb * headroom
    for pd, po in gs.candidate_grids(world):
        gb = gs.peak_memory_bytes(pd, po, g, m) / gs.GB
        ck = gs.peak_memory_bytes(pd, po, g, m, layer_ckpt=True) / gs.GB
        rows.append(dict(family="fused", grid=(pd, po), n_sub=1, ms=gs.predict_fused_ms(pd, po, g, m), gb=gb,
                         flags=f"--grid {pd} {po} --fused" + (" --checkpoint" if gb > limit >= ck else ""),
                         gb_checkpointed=ck, fits=min(gb, ck) <= limit))
        for n_sub in (2, 4, 8, 16, 32, 64, 128):
            sgb = gs.peak_memory_bytes(pd, po, g, m, n_sub, True) / gs.GB
            if sgb <= limit:
                rows.append(dict(family="streamed", grid=(pd, po), n_sub=n_sub, ms=gs.predict_streamed_ms(pd, po, n_sub, g, m), gb=sgb,
                                 flags=f"--grid {pd} {po} --fused --stream_sub {n_sub}", fits=True))
                break
    for c in gs.candidate_grids_3d(world, m.heads):
        gb = gs.peak_memory_head_bytes(*c, g, m) / gs.GB
        rows.append(dict(family="head", grid=c, n_sub=1, ms=gs.predict_head_ms(*c, g, m), gb=gb, flags="--grid %d %d %d" % c, fits=gb <= limit))
    if world > 1:
        gb = gs.peak_memory_ring_bytes(world, g, m) / gs.GB
        rows.append(dict(family="ring", grid=(world, 1), n_sub=1, ms=gs.predict_ring_ms(world, g, m), gb=gb, flags=f"--grid {world} 1 --ring",
                         fits=gb <= limit))
    rows.sort(key=lambda r: (not r["fits"], r["ms"]))
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description="predicted step time and memory of every layout for a graph on N B200s")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=None, help="a named benchmark graph instead of --nodes / --edges / --features")
    ap.add_argument("--nodes", type=int, default=None)
    ap.add_argument("--edges", type=int, default=None, help="directed edges of the graph (both directions counted)")
    ap.add_argument("--features", type=int, default=128)
    ap.add_argument("--classes", type=int, default=40)
    ap.add_argument("--exp_deg", type=int, default=4, help="expander degree of the Exphormer attention graph (0: attention over the graph edges only)")
    ap.add_argument("--token", action="store_true", help="a global token connected to every node")
    ap.add_argument("--token_dense", action="store_true", help="model the token as dense terms (train_dist --token_dense) instead of 2 n edges")
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--no_gcn", action="store_true")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--comm", default="p2p", choices=["nccl", "p2p"])
    ap.add_argument("--capacity_gb", type=float, default=gs.CAPACITY_GB)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    if args.workload:
        for k, v in WORKLOADS[args.workload].items():
            setattr(args, k, v)
    if args.nodes is None or args.edges is None:
        ap.error("give --workload or both --nodes and --edges")
    e_attn = gs.attention_edges(args.nodes, args.edges, args.exp_deg) + (2 * args.nodes if args.token else 0)
    g = gs.Graph(args.nodes, e_attn, args.edges + args.nodes, args.features, classes=args.classes, exp_deg=args.exp_deg, token=args.token)
    m = gs.Model(args.hidden, args.heads, args.layers, with_gcn=not args.no_gcn, transport=args.comm, token_dense=args.token_dense)
    rows = layouts(args.gpus, g, m, args.capacity_gb)
    if args.json:
        print(json.dumps(dict(nodes=args.nodes, attn_edges=e_attn, gpus=args.gpus, capacity_gb=args.capacity_gb, layouts=rows)))
        return rows
    print(f"graph: {args.nodes:,} nodes, {e_attn:,} attention edges, {args.features} features; model {args.layers} x {args.hidden} x {args.heads} heads; "
          f"{args.gpus} GPUs of {args.capacity_gb:.0f} GB ({gs.HEADROOM:.0%} usable), transport {args.comm}")
    print(f"{'layout':<10} {'grid':<10} {'sub-blocks':>10} {'ms / step':>11} {'GB / GPU':>10}  fits  flags")
    for r in rows:
        print(f"{r['family']:<10} {'x'.join(map(str, r['grid'])):<10} {r['n_sub']:>10} {r['ms']:>11.2f} {r['gb']:>10.2f}  {'yes' if r['fits'] else 'NO ':<4}  {r['flags']}")
    best = next((r for r in rows if r["fits"]), None)
    print("no layout fits: more GPUs, the streamed layer with more sub-blocks, or activation checkpointing" if best is None
          else f"fastest that fits: {best['family']} {'x'.join(map(str, best['grid']))} ({best['ms']:.2f} ms predicted)")
    return rows


if __name__ == "__main__":
    main()
