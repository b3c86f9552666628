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

DEFAULT_GRIDS = {1: (1, 1), 2: (2, 1), 4: (2, 2), 8: (2, 4)}


def pad_to(n, mult):
    return -(-n // mult) * mult


def exphormer_workload(name="exphormer_arxiv", grid_shape=None, device="cpu", dtype=torch.float32, seed=0, scale_down=1,
                       exp_deg=4, virtual_node=True, dropout=0.1, backend=None, layer="fused", norm="ln", stream_sub=1,
                       comm_bf16=True, heap=None, layers=None, hidden=None, heads=None, **model_kw):
    """Exphormer on a named graph: symmetrised base graph + degree-``exp_deg`` expander (both directions) + optional global
    token (edge type 2) + one self loop per node for the GCN branch.  Returns a dict with ``grid, model, x, y, masks,
    n_train, num_attn_edges, num_nodes, cfg``."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    grid_shape = tuple(grid_shape or DEFAULT_GRIDS[world])
    wl = workload_graph(name, seed=seed, scale_down=scale_down)
    cfg = wl["cfg"]
    n = wl["n"]
    n_tot = n + (1 if virtual_node else 0)                      # the token is node id n
    ei = wl["edge_index"]
    exp = keyed_expander_edges(n, exp_deg, seed=seed)
    tok = virtual_node_edges(n)[0] if virtual_node else None
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
               n_train=int(masks["train"].sum()), in_degree=degrees(ei, n)[0])
    return out
