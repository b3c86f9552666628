"""Builders that turn a named synthetic workload into (grid, local blocks, model, owned data) on every rank.

Every rank generates the same seeded global graph on the host and keeps only its own block (graphs up to a few million
nodes; larger ones go through the streaming partitioner of :mod:`gt_b200.data.partition`).  Used by ``bench.py``, the
``train_dist`` command line (``--synthetic NAME``) and the tests.
"""
import torch
import torch.distributed as dist

from ..data.expander import keyed_expander_edges
from ..data.synthetic import degrees, virtual_node_edges, workload_graph
from ..models.exphormer_dist import DistExphormer, gcn_edges_with_self_loops
from ..models.exphormer_ref import ExphormerRef
from ..parallel.grid import make_grid

DEFAULT_GRIDS = {1: (1, 1), 2: (2, 1), 4: (2, 2), 8: (4, 2)}


def pad_to(n, mult):
    return -(-n // mult) * mult


def _generate(name, seed, scale_down, device):
    """The named base graph.  Graphs of half a million nodes and more are generated on the GPU when there is one (sorting 10^8
    edges on one host core per rank would dominate a run); node data always comes back on the host.  The generators are
    deterministic per device type, so every rank still builds the same graph."""
    from ..data.synthetic import WORKLOADS
    dev = torch.device(device)
    big = WORKLOADS[name]["n"] // max(scale_down, 1) >= 500_000
    gen_dev = dev if (dev.type == "cuda" and big) else torch.device("cpu")
    wl = workload_graph(name, seed=seed, device=gen_dev, scale_down=scale_down)
    wl["x"], wl["y"] = wl["x"].cpu(), wl["y"].cpu()
    wl["masks"] = {k: m.cpu() for k, m in wl["masks"].items()}
    return wl


def exphormer_workload(name="exphormer_arxiv", grid_shape=None, device="cpu", dtype=torch.float32, seed=0, scale_down=1,
                       exp_deg=4, virtual_node=True, dropout=0.1, backend=None, layer="fused", norm="ln", stream_sub=1,
                       comm_bf16=True, heap=None, layers=None, hidden=None, heads=None, return_blocks=False, token_dense=False,
                       **model_kw):
    """Exphormer on a named graph: symmetrised base graph + degree-``exp_deg`` expander (both directions) + optional global
    token (edge type 2) + one self loop per node for the GCN branch.  ``token_dense``: the token's edges stay out of the sparse
    blocks and its row and column are computed as dense terms (``parallel/token_dense.py``; same model, same result).  Returns a
    dict with ``grid, model, x, y, masks, n_train, num_attn_edges, num_nodes, cfg``."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    grid_shape = tuple(grid_shape or DEFAULT_GRIDS[world])
    wl = _generate(name, seed, scale_down, device)
    cfg = wl["cfg"]
    n = wl["n"]
    n_tot = n + (1 if virtual_node else 0)                      # the token is node id n
    ei = wl["edge_index"]
    exp = keyed_expander_edges(n, exp_deg, seed=seed, device=ei.device)
    tok = virtual_node_edges(n)[0].to(ei.device) if virtual_node else None
    token_dense = bool(token_dense and virtual_node)
    attn_ei, attn_et = ExphormerRef.build_attention_edges(ei, exp, None if token_dense else tok)
    gcn_ei = gcn_edges_with_self_loops(ei, n_tot)
    n_pad = pad_to(n_tot, 8 * world * max(stream_sub, 1))
    grid = make_grid(grid_shape, n_tot, n_pad=n_pad).to(device)
    a_blk, a_et = grid.local_block(attn_ei, attn_et)
    g_blk, _ = grid.local_block(gcn_ei)
    dev = torch.device(device)
    backend = backend or ("cuda" if dev.type == "cuda" else "torch")
    bf16 = dtype == torch.bfloat16
    kw = dict(dropout=dropout, gnn_dropout=dropout, num_edge_types=3 if virtual_node else 2, backend=backend, norm=norm,
              fused=layer in ("fused", "streamed", "pipelined"), stream_sub=stream_sub if layer == "streamed" else 1,
              pipeline_sub=stream_sub if layer == "pipelined" else 1, ring=layer == "ring",
              comm_dtype=torch.bfloat16 if (comm_bf16 and dev.type == "cuda") else None,
              rs_dtype=torch.bfloat16 if (comm_bf16 and dev.type == "cuda" and world > 1) else None,
              kernel_dtype=torch.bfloat16 if bf16 else None, heap=heap, token_node=n if token_dense else None)
    kw.update(model_kw)
    torch.manual_seed(seed)
    model = DistExphormer(grid, g_blk.to(dev), a_blk.to(dev), a_et.to(dev), cfg["features"], hidden or cfg["hidden"], cfg["classes"],
                          layers or cfg["layers"], heads or cfg["heads"], **kw).to(dev)
    x = torch.cat([wl["x"], wl["x"].new_zeros(n_tot - n, wl["x"].shape[1])])
    y = torch.cat([wl["y"], wl["y"].new_zeros(n_tot - n)])
    masks = {k: torch.cat([m, m.new_zeros(n_tot - n)]) for k, m in wl["masks"].items()}
    out = dict(grid=grid, model=model, cfg=cfg, num_nodes=n_tot, num_attn_edges=int(attn_ei.shape[1]) + (2 * n if token_dense else 0),
               num_gcn_edges=int(gcn_ei.shape[1]), x=grid.take_owned(x).to(dtype), y=grid.take_owned(y),
               masks={k: grid.take_owned(m.to(torch.uint8)).bool() & grid.valid_mask.cpu() for k, m in masks.items()},
               n_train=int(masks["train"].sum()), in_degree=degrees(ei, n)[0].cpu())
    if return_blocks:                                          # local edge lists of this rank (tests)
        out["blocks"] = dict(attn=a_blk, attn_type=a_et, gcn=g_blk)
    return out


def exphormer_workload_streamed(name="exphormer_rmat26", grid_shape=None, device="cpu", dtype=torch.float32, seed=0, scale_down=1, exp_deg=4,
                                virtual_node=False, chunk_edges=1 << 24, dropout=0.1, backend=None, layer="streamed", norm="ln", stream_sub=1,
                                comm_bf16=True, heap=None, layers=None, hidden=None, heads=None, return_blocks=False, **model_kw):
    """:func:`exphormer_workload` for the R-MAT scale-out workload without any rank ever holding the global graph.

    Every rank walks the same seeded sequence of R-MAT edge chunks (``chunk_edges`` edges at a time), symmetrises each chunk and
    keeps the edges of ITS block only; duplicates are removed inside the block (which equals removing them globally and then
    taking the block).  Expander edges come from the per-block generator, the token's edges are written down directly, and the
    node data of the owned chunk come from per-node-block generators (:func:`gt_b200.data.synthetic.node_data_range`).  Peak
    host / device memory is one chunk plus the block, instead of the whole edge list plus its sort buffers."""
    import math

    from ..attention.csr import BlockCSR  # noqa: F401  (the model builds its CSR from the local edge lists)
    from ..data.expander import block_expander_edges
    from ..data.synthetic import WORKLOADS, node_data_range, rmat_chunks
    if name != "exphormer_rmat26":
        raise ValueError("the streamed builder generates the R-MAT workload 'exphormer_rmat26'")
    world = dist.get_world_size() if dist.is_initialized() else 1
    grid_shape = tuple(grid_shape or DEFAULT_GRIDS[world])
    cfg = dict(WORKLOADS[name])
    sc = 26 - int(math.log2(scale_down)) if scale_down > 1 else 26
    n = 1 << sc
    cfg["n"] = n
    n_tot = n + (1 if virtual_node else 0)
    n_pad = pad_to(n_tot, 8 * world * max(stream_sub, 1))
    grid = make_grid(grid_shape, n_tot, n_pad=n_pad).to(device)
    dev = torch.device(device)
    gen_dev = dev if dev.type == "cuda" else torch.device("cpu")
    n_cols = grid.n_col_block
    keys = []
    for chunk in rmat_chunks(sc, (16 << sc) // 2, seed=seed, device=gen_dev, chunk=chunk_edges):
        both = torch.cat([chunk, chunk.flip(0)], dim=1)
        loc, _ = grid.local_block(both)
        keys.append(torch.unique(loc[1] * n_cols + loc[0]))                  # (row-local dst, col-local src) as one key
    key = torch.unique(torch.cat(keys)) if keys else torch.zeros(0, dtype=torch.long, device=gen_dev)
    base = torch.stack([key % n_cols, key // n_cols])                          # local (src, dst), sorted by (dst, src)
    exp = block_expander_edges(grid, n, exp_deg, seed=seed, device=gen_dev) if exp_deg > 0 else base.new_zeros(2, 0)
    parts, types = [base, exp], [0, 1]
    if virtual_node:                                                           # token id n: edges (i -> n) and (n -> i) for i < n
        r_lo_hi, (c_lo, c_hi) = grid.row_block_ranges(), grid.col_block_range()
        tok_in_rows = any(lo <= n < hi for lo, hi in r_lo_hi)
        tok_in_cols = c_lo <= n < c_hi
        t_src, t_dst = [], []
        if tok_in_rows:                                                        # the token attends to the nodes of my column block
            src = torch.arange(c_lo, min(c_hi, n), device=gen_dev)
            t_src.append(src); t_dst.append(torch.full_like(src, n))
        if tok_in_cols:                                                        # the nodes of my row block attend to the token
            dst = torch.cat([torch.arange(lo, min(hi, n), device=gen_dev) for lo, hi in r_lo_hi]) if any(lo < n for lo, _ in r_lo_hi) \
                else torch.zeros(0, dtype=torch.long, device=gen_dev)
            t_src.append(torch.full_like(dst, n)); t_dst.append(dst)
        if t_src:
            gs_, gd_ = torch.cat(t_src), torch.cat(t_dst)
            parts.append(torch.stack([grid.global_to_col_local(gs_), grid.global_to_row_local(gd_)]))
            types.append(2)
    a_blk = torch.cat(parts, dim=1)
    a_et = torch.cat([torch.full((p.shape[1],), t, dtype=torch.long, device=gen_dev) for p, t in zip(parts, types)])
    # GCN block: base edges + one self loop for every node that is both one of my rows and one of my columns
    cb_lo, cb_hi = grid.col_block_range()
    loops_g = torch.cat([torch.arange(max(lo, cb_lo), max(min(hi, cb_hi, n_tot), max(lo, cb_lo)), device=gen_dev)
                         for lo, hi in grid.row_block_ranges()] + [torch.zeros(0, dtype=torch.long, device=gen_dev)])
    loops = torch.stack([grid.global_to_col_local(loops_g), grid.global_to_row_local(loops_g)])
    g_blk = torch.cat([base, loops], dim=1)
    backend = backend or ("cuda" if dev.type == "cuda" else "torch")
    bf16 = dtype == torch.bfloat16
    kw = dict(dropout=dropout, gnn_dropout=dropout, num_edge_types=3 if virtual_node else 2, backend=backend, norm=norm,
              fused=layer in ("fused", "streamed", "pipelined"), stream_sub=stream_sub if layer == "streamed" else 1,
              pipeline_sub=stream_sub if layer == "pipelined" else 1,
              comm_dtype=torch.bfloat16 if (comm_bf16 and dev.type == "cuda") else None,
              rs_dtype=torch.bfloat16 if (comm_bf16 and dev.type == "cuda" and world > 1) else None,
              kernel_dtype=torch.bfloat16 if bf16 else None, heap=heap)
    kw.update(model_kw)
    torch.manual_seed(seed)
    model = DistExphormer(grid, g_blk.to(dev), a_blk.to(dev), a_et.to(dev), cfg["features"], hidden or cfg["hidden"], cfg["classes"],
                          layers or cfg["layers"], heads or cfg["heads"], **kw).to(dev)
    lo, hi = grid.owned_range()
    x_o, y_o, m_o = node_data_range(lo, min(hi, n), cfg["features"], cfg["classes"], (0.01, 0.01, 0.98), seed=seed + 17, device="cpu")

    def pad_rows(t):
        out = t.new_zeros((grid.chunk,) + tuple(t.shape[1:]))
        out[:t.shape[0]] = t
        return out

    valid = grid.valid_mask.cpu()
    masks = {k: pad_rows(v) & valid for k, v in m_o.items()}
    counts = torch.tensor([a_blk.shape[1], g_blk.shape[1], int(masks["train"].sum())], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(counts)
    p_heads = grid_shape[2] if len(grid_shape) == 3 else 1
    out = dict(grid=grid, model=model, cfg=cfg, num_nodes=n_tot, num_attn_edges=int(counts[0].item()) // p_heads,
               num_gcn_edges=int(counts[1].item()) // p_heads, x=pad_rows(x_o).to(dtype), y=pad_rows(y_o), masks=masks,
               n_train=int(counts[2].item()), in_degree=None)
    if return_blocks:
        out["blocks"] = dict(attn=a_blk, attn_type=a_et, gcn=g_blk)
    return out


def variant_workload(model="unimp", name=None, grid_shape=None, device="cpu", dtype=torch.float32, seed=0, scale_down=1,
                     dropout=0.3, backend=None, comm_bf16=False, khop=False, max_two_hop=64, label_input=False,
                     layers=None, hidden=None, heads=None, max_degree=None, ffn_mult=2, checkpoint=False):
    """UniMP or Graphormer-node on a named graph (defaults: ``unimp_products`` / ``graphormer_rmat``).  ``khop``: the 2-hop mask
    with distance-bucket bias and in/out-degree embeddings (clipped at ``max_degree``, default 512); otherwise the 1-hop mask
    with a global token.  Returns the same dict as ``exphormer_workload`` plus ``degree`` / ``out_degree`` of the owned rows."""
    from ..models import gt_variants as gv
    world = dist.get_world_size() if dist.is_initialized() else 1
    grid_shape = tuple(grid_shape or DEFAULT_GRIDS[world])
    name = name or ("unimp_products" if model == "unimp" else "graphormer_rmat")
    wl = _generate(name, seed, scale_down, device)
    cfg, n, ei = wl["cfg"], wl["n"], wl["edge_index"]
    dev = torch.device(device)
    backend = backend or ("cuda" if dev.type == "cuda" else "torch")
    token = model == "graphormer" and not khop
    n_tot = n + (1 if token else 0)
    if model == "unimp":
        a_ei, a_et = gv.typed_graph_edges(ei, n)
        nb_type, n_types = 0, 2
    elif khop:
        a_ei, a_et = gv.khop_typed_edges(ei, n, max_two_hop=max_two_hop, seed=seed)
        nb_type, n_types = 1, 3
    else:
        a_ei, a_et = gv.graphormer_edges(ei, n)
        nb_type, n_types = 0, 4
    n_pad = pad_to(n_tot + (0 if not token else 0), 8 * world)
    if token and n_pad == n_tot:
        n_pad += 8 * world
    grid = make_grid(grid_shape, n_tot if not token else n, n_pad=n_pad).to(device)
    b_ei, b_et = grid.local_block(a_ei, a_et)
    kw = dict(model=model, dropout=dropout, backend=backend, checkpoint=checkpoint,
              comm_dtype=torch.bfloat16 if (comm_bf16 and dev.type == "cuda") else None,
              rs_dtype=torch.bfloat16 if (comm_bf16 and dev.type == "cuda" and world > 1) else None)
    if model == "unimp":
        kw.update(num_classes_label=cfg["classes"] if label_input else None)
    else:
        kw.update(max_degree=max_degree or (512 if khop else 64), num_edge_types=n_types, out_degree=khop, ffn_mult=ffn_mult,
                  token_row=gv.token_owned_row(grid, n) if token else None)
    torch.manual_seed(seed)
    net = gv.DistGTVariant(grid, b_ei.to(dev), b_et.to(dev), cfg["features"], hidden or cfg["hidden"], cfg["classes"],
                           layers or cfg["layers"], heads or cfg["heads"], **kw).to(dev)
    rows = n_pad
    x = torch.zeros(rows, wl["x"].shape[1]); x[:n] = wl["x"]
    y = torch.zeros(rows, dtype=torch.long); y[:n] = wl["y"]
    masks = {}
    for k, m in wl["masks"].items():
        mm = torch.zeros(rows, dtype=torch.bool); mm[:n] = m
        masks[k] = grid.take_owned(mm.to(torch.uint8)).bool()
    out = dict(grid=grid, model=net, cfg=cfg, num_nodes=n_tot, num_attn_edges=int(a_ei.shape[1]), x=grid.take_owned(x).to(dtype),
               y=grid.take_owned(y), masks=masks, n_train=int(wl["masks"]["train"].sum()))
    if model == "graphormer":
        d_in, d_out = gv.owned_degrees(grid, b_ei.to(dev), b_et.to(dev), dev, neighbour_type=nb_type)
        out.update(degree=d_in, out_degree=d_out if khop else None)
    return out
