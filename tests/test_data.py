"""Expander generation, synthetic graphs, partitioner + loaders (pure host, no process group)."""
import os

import pytest

import torch

from gt_b200.data.expander import KeyedPermutation, block_expander_edges, keyed_expander_edges
from gt_b200.data.loader import load_partition, read_meta
from gt_b200.data.partition import partition_2d
from gt_b200.data.synthetic import chung_lu, degrees, khop_edges, rmat, symmetrize, workload_graph
from gt_b200.parallel.grid import BlockGrid


def test_keyed_permutation_is_bijection_for_odd_sizes():
    for n in (1, 2, 7, 1000, 4097):
        img = KeyedPermutation(n, seed=3, index=1)(torch.arange(n))
        assert img.unique().numel() == n and int(img.max()) == n - 1


def test_block_expander_equals_global_on_several_grids():
    n, deg = 1013, 3
    glob = keyed_expander_edges(n, deg, seed=5)
    key = lambda e: torch.unique(e[1] * 4096 + e[0])          # noqa: E731
    for shape in ((2, 2, 1), (4, 1, 1), (1, 3, 1), (2, 1, 2)):
        world = shape[0] * shape[1] * shape[2]
        got = []
        for rank in range(world):
            g = BlockGrid.virtual(shape[0], shape[1], n, rank, p_heads=shape[2])
            loc = block_expander_edges(g, n, deg, seed=5)
            ref_loc, _ = g.local_block(glob)
            assert torch.equal(key(loc), key(ref_loc)), (shape, rank)
            got.append(loc.shape[1])
        assert sum(got) == glob.shape[1] * shape[2]             # head-group ranks hold the same block


def test_synthetic_generators_shapes_and_determinism():
    a = chung_lu(2000, 9000, 2.1, seed=1)
    assert torch.equal(a, chung_lu(2000, 9000, 2.1, seed=1)) and int(a.max()) < 2000
    ind, _ = degrees(symmetrize(a, 2000), 2000)
    assert ind.max() > 20 * ind.float().mean()                   # heavy tail
    r = rmat(10, 5000, seed=2)
    assert int(r.max()) < 1024 and r.shape[1] > 4000
    ei, bucket = khop_edges(symmetrize(r, 1024), 1024)
    assert set(bucket.unique().tolist()) == {0, 1, 2}
    wl = workload_graph("cpu_small")
    assert wl["n"] == 2000 and wl["x"].shape == (2000, 32)


def test_partition_roundtrip_and_resume(tmp_path):
    wl = workload_graph("cpu_small", seed=1)
    n, ei = wl["n"], wl["edge_index"]
    w = torch.rand(ei.shape[1])
    out = str(tmp_path / "part")
    meta = partition_2d(wl["x"], wl["y"], wl["masks"], ei, 10, out, p_part=4, edge_weight=w, pad_multiple=8, log=lambda *a: None)
    assert read_meta(out)["n_pad"] == meta["n_pad"] and meta["n_pad"] % 8 == 0
    os.remove(os.path.join(out, "blocks", "row_2.done"))          # an interrupted run: row 2 is redone, the others are skipped
    logs = []
    partition_2d(wl["x"], wl["y"], wl["masks"], ei, 10, out, p_part=4, edge_weight=w, pad_multiple=8, log=logs.append)
    assert sum("skipped" in l for l in logs) == 3
    for shape in ((2, 2), (1, 2), (8, 1), (2, 1, 2)):
        world = 1
        for s in shape:
            world *= s
        tot_e, tot_x = 0, 0
        for rank in range(world):
            g = BlockGrid.virtual(shape[0], shape[1], n, rank, p_heads=shape[2] if len(shape) == 3 else 1, n_pad=meta["n_pad"])
            part = load_partition(out, g, "cpu")
            ref_ei, _, ref_w = g.local_block(ei, None, w)
            k = lambda e: e[1] * 100000 + e[0]                   # noqa: E731
            o1, o2 = torch.argsort(k(part["edge_index"])), torch.argsort(k(ref_ei))
            assert torch.equal(part["edge_index"][:, o1], ref_ei[:, o2]) and torch.allclose(part["weight"][o1], ref_w[o2])
            assert torch.equal(part["x"], g.take_owned(wl["x"])) and torch.equal(part["y"], g.take_owned(wl["y"]))
            tot_e += part["num_local_edges"]
            tot_x += int(part["masks"]["train"].sum())
        assert tot_e == ei.shape[1] * (shape[2] if len(shape) == 3 else 1)
        assert tot_x == int(wl["masks"]["train"].sum())


def test_plexus_layout_loader(tmp_path):
    """A partition in the Plexus layout (destination-first edge files, features split in column pieces) loads onto grids whose
    chunks differ from the partition's, with the same blocks and node arrays as a direct split of the global graph."""
    from gt_b200.data.loader import grid_n_pad, load_plexus_partition, read_plexus_meta
    wl = workload_graph("cpu_small", seed=2)
    n, ei, x, y, masks = wl["n"], wl["edge_index"], wl["x"], wl["y"], wl["masks"]
    w = torch.rand(ei.shape[1])
    p = 3
    chunk = -(-n // p)
    f = x.shape[1]
    out = tmp_path / "plexus"
    for sub in ("edge_index/0", "input_features", "output_labels/0", "masks/train/0", "masks/val/0", "masks/test/0"):
        os.makedirs(out / sub)
    torch.save((n, f, int(y.max()) + 1), out / "metadata.pt")
    pieces = [(j * f // p, (j + 1) * f // p) for j in range(p)]
    for i in range(p):
        a, b = i * chunk, min(n, (i + 1) * chunk)
        torch.save(y[a:b].view(-1, 1), out / "output_labels" / "0" / f"{i}.pt")
        for j, (c0, c1) in enumerate(pieces):
            torch.save(x[a:b, c0:c1].clone(), out / "input_features" / f"{i}_{j}.pt")
        for k, s in (("train", "train"), ("valid", "val"), ("test", "test")):
            torch.save(masks[k][a:b].clone(), out / "masks" / s / "0" / f"{i}.pt")
        for j in range(p):                                   # file "{dst chunk}_{src chunk}": rows (dst, src), global ids
            sel = (ei[1] // chunk == i) & (ei[0] // chunk == j)
            torch.save((ei[:, sel].flip(0).clone(), w[sel].clone()), out / "edge_index" / "0" / f"{i}_{j}.pt")
    meta = read_plexus_meta(str(out))
    assert meta["layout"] == "plexus" and meta["p_part"] == p and meta["chunk"] == chunk and meta["num_features"] == f
    for shape in ((2, 2), (1, 2), (4, 1), (2, 1, 2)):
        world = 1
        for s in shape:
            world *= s
        n_pad = grid_n_pad(meta, world, 8)
        assert n_pad % world == 0 and n_pad % 8 == 0 and n_pad >= n
        tot_e = tot_train = 0
        for rank in range(world):
            g = BlockGrid.virtual(shape[0], shape[1], n, rank, p_heads=shape[2] if len(shape) == 3 else 1, n_pad=n_pad)
            part = load_plexus_partition(str(out), g, "cpu")
            ref_ei, _, ref_w = g.local_block(ei, None, w)
            k = lambda e: e[1] * 100000 + e[0]                   # noqa: E731
            o1, o2 = torch.argsort(k(part["edge_index"])), torch.argsort(k(ref_ei))
            assert torch.equal(part["edge_index"][:, o1], ref_ei[:, o2]) and torch.allclose(part["weight"][o1], ref_w[o2])
            assert torch.equal(part["x"], g.take_owned(x)) and torch.equal(part["y"], g.take_owned(y))
            tot_e += part["num_local_edges"]
            tot_train += int(part["masks"]["train"].sum())
        assert tot_e == ei.shape[1] * (shape[2] if len(shape) == 3 else 1)
        assert tot_train == int(masks["train"].sum()) * 1
    os.makedirs(out / "edge_index" / "1")
    with pytest.raises(ValueError):
        read_plexus_meta(str(out))                            # two node orders: refused


def _streamed_workload_worker(rank, world, shape):
    """The streamed builder yields, block by block, the edge sets of the builder that materialises the global graph (same R-MAT
    chunk sequence), and node data that depend only on the node id."""
    import torch.distributed as dist
    from gt_b200.data.synthetic import node_data_range
    from gt_b200.train.workloads import exphormer_workload, exphormer_workload_streamed
    kw = dict(name="exphormer_rmat26", grid_shape=shape, scale_down=1 << 15, virtual_node=True, layers=1, hidden=16, heads=2,
              return_blocks=True)
    layer = "fused" if len(shape) == 2 else "head"
    a = exphormer_workload(layer=layer, **kw)
    b = exphormer_workload_streamed(layer=layer, chunk_edges=1 << 26, **kw)

    def keyset(ei, et=None):
        k = ei[1] * 10_000_000 + ei[0] * 10 + (et if et is not None else 0)
        return torch.unique(k)

    assert a["num_nodes"] == b["num_nodes"] == 2049 and a["grid"].n_pad == b["grid"].n_pad
    assert torch.equal(keyset(a["blocks"]["attn"], a["blocks"]["attn_type"]), keyset(b["blocks"]["attn"].cpu(), b["blocks"]["attn_type"].cpu()))
    assert a["blocks"]["attn"].shape[1] == b["blocks"]["attn"].shape[1]
    assert torch.equal(keyset(a["blocks"]["gcn"]), keyset(b["blocks"]["gcn"].cpu())) and a["blocks"]["gcn"].shape[1] == b["blocks"]["gcn"].shape[1]
    assert a["num_attn_edges"] == b["num_attn_edges"] and a["num_gcn_edges"] == b["num_gcn_edges"]
    # a smaller chunk size walks a different random sequence: another graph of the same family, same bookkeeping
    c = exphormer_workload_streamed(layer=layer, chunk_edges=1 << 12, **kw)
    assert 0.8 < c["num_attn_edges"] / b["num_attn_edges"] < 1.25
    lo, hi = b["grid"].owned_range()
    x_ref, y_ref, _ = node_data_range(0, 2048, b["cfg"]["features"], b["cfg"]["classes"], (0.01, 0.01, 0.98), seed=17)
    nv = max(min(hi, 2048) - lo, 0)
    assert torch.equal(b["x"][:nv], x_ref[lo:lo + nv]) and torch.equal(b["y"][:nv], y_ref[lo:lo + nv])
    tot = torch.tensor([float(b["masks"]["train"].sum())], dtype=torch.float64)
    dist.all_reduce(tot)
    assert int(tot.item()) == b["n_train"]
    out = b["model"](b["x"])                                  # the model runs on the streamed blocks
    assert out.shape[0] == b["grid"].chunk and torch.isfinite(out).all()


@pytest.mark.parametrize("shape", [(2, 2), (1, 2, 2)], ids=["2x2", "1x2x2"])
def test_streamed_workload_matches_global_builder(shape):
    from dist_utils import run_dist
    run_dist(_streamed_workload_worker, 4, shape)
