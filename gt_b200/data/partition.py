"""Streaming 2D partitioner: cut a full graph into ``p x p`` edge blocks and ``p`` node chunks in ONE node-id space.

Directory layout (the one the reference's loader reads, ``gt3d/gt3d/data/partition.py:1-12``, so partitions are
interchangeable):

    meta.json                     num_nodes, num_features, num_classes, p_part, chunk, n_pad, num_edges, has_weight, self_loops
    blocks/{i}_{j}.pt             (edge_index [2, E_ij] global ids, weight [E_ij] | None), src in chunk i, dst in chunk j
    blocks/row_{i}.done           JSON marker: block row i is complete (resume point)
    x/{i}.pt  y/{i}.pt  mask_{train,val,test}/{i}.pt     per-node arrays of chunk i (last chunk unpadded)

``n_pad`` is a multiple of ``lcm(p_part, pad_multiple)`` so that every grid whose size divides ``pad_multiple`` gets whole
chunks.  Edges are bucketed one source-chunk row at a time (peak memory: the edge list plus one row), every file is written
to a temporary name and renamed (a file that exists is complete), and finished rows are skipped on restart.

    python -m gt_b200.data.partition --synthetic exphormer_arxiv --out /data/arxiv_p8 --p_part 8
    python -m gt_b200.data.partition --src graph.pt --out DIR --p_part 16
"""
import argparse
import json
import math
import os

import torch


def _atomic_save(obj, path):
    tmp = f"{path}.tmp{os.getpid()}"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def _atomic_json(obj, path):
    tmp = f"{path}.tmp{os.getpid()}"
    with open(tmp, "w") as f:
        json.dump(obj, f, indent=1)
    os.replace(tmp, path)


def padded_size(n, p_part, pad_multiple):
    unit = p_part * pad_multiple // math.gcd(p_part, pad_multiple)
    return -(-n // unit) * unit


def partition_2d(x, y, masks, edge_index, num_classes, out_dir, p_part, edge_weight=None, pad_multiple=4096, log=print):
    """``masks``: dict with keys train / val (or valid) / test.  ``edge_index``: [2, E] (src, dst) global ids."""
    n, f = x.shape
    n_pad = padded_size(n, p_part, pad_multiple)
    chunk = n_pad // p_part
    for sub in ("blocks", "x", "y", "mask_train", "mask_val", "mask_test"):
        os.makedirs(os.path.join(out_dir, sub), exist_ok=True)
    mk = {"train": masks["train"], "val": masks.get("val", masks.get("valid")), "test": masks["test"]}
    for i in range(p_part):
        lo, hi = i * chunk, min((i + 1) * chunk, n)
        lo = min(lo, n)
        fx = os.path.join(out_dir, "x", f"{i}.pt")
        if not os.path.exists(fx):
            _atomic_save(x[lo:hi].clone(), fx)
        _atomic_save(y.view(-1)[lo:hi].clone(), os.path.join(out_dir, "y", f"{i}.pt"))
        for name, m in mk.items():
            _atomic_save(m[lo:hi].clone(), os.path.join(out_dir, f"mask_{name}", f"{i}.pt"))
    src_chunk = torch.div(edge_index[0], chunk, rounding_mode="floor")
    order = torch.argsort(src_chunk, stable=True)                 # one pass groups the edges by source chunk
    row_ptr = torch.zeros(p_part + 1, dtype=torch.long)
    torch.cumsum(torch.bincount(src_chunk, minlength=p_part), 0, out=row_ptr[1:])
    loops_total, counts = 0, []
    for i in range(p_part):
        marker = os.path.join(out_dir, "blocks", f"row_{i}.done")
        if os.path.exists(marker):
            with open(marker) as fh:
                done = json.load(fh)
            counts += done["counts"]
            loops_total += int(done["self_loops"])
            log(f"  block row {i + 1}/{p_part} already complete, skipped")
            continue
        sel = order[row_ptr[i]:row_ptr[i + 1]]
        ei_i = edge_index[:, sel]
        w_i = edge_weight[sel] if edge_weight is not None else None
        dst_chunk = torch.div(ei_i[1], chunk, rounding_mode="floor")
        o2 = torch.argsort(dst_chunk, stable=True)
        ei_i, w_i = ei_i[:, o2], (w_i[o2] if w_i is not None else None)
        cnt = torch.bincount(dst_chunk, minlength=p_part)
        off = torch.zeros(p_part + 1, dtype=torch.long)
        torch.cumsum(cnt, 0, out=off[1:])
        loops = 0
        for j in range(p_part):
            a, b = int(off[j]), int(off[j + 1])
            blk = ei_i[:, a:b].clone()
            loops += int((blk[0] == blk[1]).sum())
            _atomic_save((blk, w_i[a:b].clone() if w_i is not None else None), os.path.join(out_dir, "blocks", f"{i}_{j}.pt"))
        _atomic_json(dict(counts=cnt.tolist(), self_loops=loops), marker)
        counts += cnt.tolist()
        loops_total += loops
        log(f"  wrote block row {i + 1}/{p_part}")
    meta = dict(num_nodes=int(n), num_features=int(f), num_classes=int(num_classes), p_part=int(p_part), chunk=int(chunk),
                n_pad=int(n_pad), num_edges=int(edge_index.shape[1]), has_weight=edge_weight is not None, self_loops=int(loops_total))
    _atomic_json(meta, os.path.join(out_dir, "meta.json"))
    return meta


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=None, help=".pt file holding an object (or (object, (num_classes,))) with x, y, edge_index, "
                                                "train_mask, val_mask, test_mask and optionally edge_weight")
    ap.add_argument("--synthetic", default=None, help="name of a synthetic workload (gt_b200.data.synthetic.WORKLOADS)")
    ap.add_argument("--scale_down", type=int, default=1)
    ap.add_argument("--gcn_weights", action="store_true", help="store self loops and symmetric GCN weights with the edges")
    ap.add_argument("--out", required=True)
    ap.add_argument("--p_part", type=int, default=16)
    ap.add_argument("--pad_multiple", type=int, default=4096)
    args = ap.parse_args()
    if args.synthetic:
        from .synthetic import workload_graph
        wl = workload_graph(args.synthetic, scale_down=args.scale_down)
        x, y, masks, ei, nc, w = wl["x"], wl["y"], wl["masks"], wl["edge_index"], wl["num_classes"], None
    else:
        obj = torch.load(args.src, weights_only=False)
        data, nc = (obj[0], int(obj[1][0] if isinstance(obj[1], (tuple, list)) else obj[1])) if isinstance(obj, (tuple, list)) \
            else (obj, int(obj.y.max()) + 1)
        x, y, ei, w = data.x, data.y, data.edge_index, getattr(data, "edge_weight", None)
        masks = dict(train=data.train_mask, val=data.val_mask, test=data.test_mask)
    if args.gcn_weights:
        from ..models.exphormer_ref import gcn_norm
        ei, w = gcn_norm(ei, x.shape[0], torch.float32)
    print("meta:", partition_2d(x, y, masks, ei, nc, args.out, args.p_part, w, args.pad_multiple), flush=True)


if __name__ == "__main__":
    main()
