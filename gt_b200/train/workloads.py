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
                       comm_bf16=True, heap=None, layers=None, hidden=None, heads=None, **model_kw):
    """Exphormer on a named graph: symmetrised base graph + degree-``exp_deg`` expander (both directions) + optional global
    token (edge type 2) + one self loop per node for the GCN branch.  Returns a dict with ``grid, model, x, y, masks,
    n_train, num_attn_edges, num_nodes, cfg``."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    grid_shape = tuple(grid_shape or DEFAULT_GRIDS[world])
    wl = _generate(name, seed, scale_down, device)
    cfg = wl["cfg"]
    n = wl["n"]
    n_tot = n + (1 if virtual_node else 0)                      # the token is node id n
    ei = wl["edge_index"]
    exp = keyed_expander_edges(n, exp_deg, seed=seed, device=ei.device)
    tok = virtual_node_edges(n)[0].to(ei.device) if virtual_node else None
    attn_ei, attn_et = ExphormerRef.build_attention_edges(ei, exp, tok)
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
              kernel_dtype=torch.bfloat16 if bf16 else None, heap=heap)
    kw.update(model_kw)
    torch.manual_seed(seed)
    model = DistExphormer(grid, g_blk.to(dev), a_blk.to(dev), a_et.to(dev), cfg["features"], hidden or cfg["hidden"], cfg["classes"],
                          layers or cfg["layers"], heads or cfg["heads"], **kw).to(dev)
    x = torch.cat([wl["x"], wl["x"].new_zeros(n_tot - n, wl["x"].shape[1])])
    y = torch.cat([wl["y"], wl["y"].new_zeros(n_tot - n)])
    masks = {k: torch.cat([m, m.new_zeros(n_tot - n)]) for k, m in wl["masks"].items()}
    out = dict(grid=grid, model=model, cfg=cfg, num_nodes=n_tot, num_attn_edges=int(attn_ei.shape[1]), num_gcn_edges=int(gcn_ei.shape[1]),
               x=grid.take_owned(x).to(dtype), y=grid.take_owned(y),
               masks={k: grid.take_owned(m.to(torch.uint8)).bool() & grid.valid_mask.cpu() for k, m in masks.items()},
               n_train=int(masks["train"].sum()), in_degree=degrees(ei, n)[0].cpu())
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
