"""Load one rank's share of a partition directory.

Two on-disk layouts are understood, both through one reader that only needs "which file holds the edges from node chunk i
to node chunk j" and "which files hold the per-node arrays of chunk i":

* the native layout written by :mod:`gt_b200.data.partition` (identical to the reference's, ``gt3d/gt3d/data/loader.py``);
* the Plexus layout (``metadata.pt``, ``edge_index/0/{i}_{j}.pt`` with destination-first edges, features split in ``p``
  column pieces: ``gt3d/gt3d/data/plexus_loader.py:1-16``).

The grid's chunks need not equal the partition's: a grid chunk may be a union or a sub-range of partition chunks as long as
the grid uses the partition's ``n_pad`` (native) or a compatible padding (Plexus, ``grid_n_pad``).  ``load_partition`` returns
``x, y, masks`` of the owned chunk (zero padded), the local block ``edge_index`` as (col-local src, row-local dst),
``weight`` and ``num_local_edges``.
"""
import json
import math
import os

import torch


def read_meta(part_dir):
    """Metadata of either layout (``layout`` key: 'native' or 'plexus')."""
    native = os.path.join(part_dir, "meta.json")
    if os.path.exists(native):
        with open(native) as f:
            meta = json.load(f)
        meta["layout"] = "native"
        return meta
    n, f, c = torch.load(os.path.join(part_dir, "metadata.pt"), weights_only=False)
    if os.path.isdir(os.path.join(part_dir, "edge_index", "1")):
        raise ValueError("double-permutation Plexus partitions carry two node orders and cannot be used")
    p = len([x for x in os.listdir(os.path.join(part_dir, "output_labels", "0")) if x.endswith(".pt")])
    chunk = -(-int(n) // p)
    return dict(num_nodes=int(n), num_features=int(f), num_classes=int(c), p_part=p, chunk=chunk, n_pad=chunk * p, has_weight=True,
                num_edges=None, layout="plexus")


def read_plexus_meta(part_dir):
    return read_meta(part_dir)


def grid_n_pad(meta, world, multiple=1):
    """Padded node count for a grid of ``world`` ranks over a Plexus partition."""
    m = math.lcm(world, multiple)
    return -(-meta["num_nodes"] // m) * m


class _Files:
    def __init__(self, part_dir, meta, src_first=True):
        self.dir, self.meta, self.plexus, self.src_first = part_dir, meta, meta["layout"] == "plexus", src_first

    def _ld(self, *parts):
        return torch.load(os.path.join(self.dir, *parts), weights_only=False)

    def node_arrays(self, i, a, b):
        if not self.plexus:
            x = self._ld("x", f"{i}.pt")[a:b]
            y = self._ld("y", f"{i}.pt")[a:b]
            ms = {k: self._ld(f"mask_{s}", f"{i}.pt")[a:b] for k, s in (("train", "train"), ("valid", "val"), ("test", "test"))}
            return x, y, ms
        p = self.meta["p_part"]
        x = torch.cat([self._ld("input_features", f"{i}_{j}.pt")[a:b] for j in range(p)], dim=1)
        y = self._ld("output_labels", "0", f"{i}.pt")[a:b].view(-1)
        ms = {k: self._ld("masks", s, "0", f"{i}.pt")[a:b] for k, s in (("train", "train"), ("valid", "val"), ("test", "test"))}
        return x, y, ms

    def block(self, i, j):
        """Edges with source in chunk i and destination in chunk j as ((src, dst), weight)."""
        if not self.plexus:
            return self._ld("blocks", f"{i}_{j}.pt")
        name = f"{i}_{j}.pt" if self.src_first else f"{j}_{i}.pt"
        ei, w = self._ld("edge_index", "0", name)
        return (ei if self.src_first else ei.flip(0)), w


def _chunks(lo, hi, size, limit):
    return [c for c in range(lo // size, -(-hi // size)) if c < limit]


def load_partition(part_dir, grid, device, load_weights=True, src_first=None):
    meta = read_meta(part_dir)
    plexus = meta["layout"] == "plexus"
    files = _Files(part_dir, meta, src_first=(not plexus) if src_first is None else src_first)
    pc, p, n = meta["chunk"], meta["p_part"], meta["num_nodes"]
    if not plexus and grid.n_pad != meta["n_pad"]:
        raise ValueError(f"grid n_pad {grid.n_pad} must equal the partition's {meta['n_pad']}")
    lo, hi = grid.owned_range()
    xs, ys, ms = [], [], {"train": [], "valid": [], "test": []}
    for i in _chunks(lo, min(hi, n), pc, p):
        a, b = max(lo, i * pc) - i * pc, min(hi, (i + 1) * pc, n) - i * pc
        if b <= a:
            continue
        x_i, y_i, m_i = files.node_arrays(i, a, b)
        xs.append(x_i); ys.append(y_i)
        for k in ms:
            ms[k].append(m_i[k])

    def pad_rows(parts, empty):
        t = torch.cat(parts) if parts else empty
        out = t.new_zeros((grid.chunk,) + tuple(t.shape[1:]))
        out[:t.shape[0]] = t
        return out

    f = meta["num_features"]
    x = pad_rows(xs, torch.zeros(0, f)).to(device)
    y = pad_rows(ys, torch.zeros(0, dtype=torch.long)).to(device)
    valid = grid.valid_mask.to(device)
    masks = {k: pad_rows(v, torch.zeros(0, dtype=torch.bool)).to(device) & valid for k, v in ms.items()}
    c_lo, c_hi = grid.col_block_range()
    src_chunks = _chunks(c_lo, min(c_hi, n) if plexus else c_hi, pc, p)
    dst_chunks = sorted({c for rlo, rhi in grid.row_block_ranges() for c in _chunks(rlo, min(rhi, n) if plexus else rhi, pc, p)})
    eis, ws = [], []
    for i in src_chunks:
        for j in dst_chunks:
            ei, w = files.block(i, j)
            eis.append(ei)
            if load_weights and w is not None:
                ws.append(w)
    ei = torch.cat(eis, dim=1) if eis else torch.zeros(2, 0, dtype=torch.long)
    w = torch.cat(ws) if ws else None
    keep = (grid.owner_of(ei[1])[0] == grid.r) & (grid.owner_of(ei[0])[1] == grid.c)
    ei = ei[:, keep]
    w = w[keep] if w is not None else None
    local = torch.stack([grid.global_to_col_local(ei[0]), grid.global_to_row_local(ei[1])]).to(device)
    return dict(meta=meta, x=x, y=y, masks=masks, edge_index=local, weight=w.to(device) if w is not None else None,
                num_local_edges=int(ei.shape[1]))


load_plexus_partition = load_partition
