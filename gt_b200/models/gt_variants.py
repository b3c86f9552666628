"""UniMP and Graphormer-node on the block-distributed attention operator.

UniMP (TransformerConv with gated residual and masked label prediction): mask = graph edges + self loops, dot-product
scores, softmax; per layer ``out = beta W_r x + (1 - beta) Attn(x)``, ``beta = sigmoid(W_g [r | o | r - o])``, then
LayerNorm + ReLU + dropout.  Labels of a random share of the training nodes may be fed as an input embedding.

Graphormer-node: pre-LayerNorm transformer blocks, dot-product scores plus a learnable bias per relation type and head,
softmax, GELU FFN, degree (centrality) embeddings added to the input.  Two masks are provided:
``graphormer_edges`` — 1-hop edges, self loops and a global token (types 0 neighbour, 1 self, 2 node->token,
3 token->node; the mask of the reference, ``gt3d/gt3d/models/gt_variants.py:35-57``) — and ``khop_typed_edges`` — the
2-hop neighbourhood with the shortest-path bucket {0, 1, 2} as the relation type, the mask of the 1M-node R-MAT
workload.  ``max_degree`` clips the degree embeddings (64 in the reference, 512 in that workload) and
``out_degree=True`` adds a second table for the out-degree.

The single-process classes (``UniMPRef``, ``GraphormerNodeRef``) are the fp64 oracles and fix the state-dict names; the
distributed layers use the fused-communication form on a 2D grid (gather x once per block, local projections,
unnormalised partials, one reduce-scatter) and the head-parallel form on a 3D grid (owner projects, Ulysses
all-to-all, head-slice gathers), which the reference does not have for these two models.
"""
import math

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..data.synthetic import add_self_loops, khop_edges, virtual_node_edges
from ..ops import functional as K
from ..parallel.attention import AttentionBlock, DistAttentionPartial, DistHeadSparseAttention, combine_partials
from ..parallel.collectives import all_gather_rows
from ..parallel.grid import group_size

ET_NEIGHBOUR, ET_SELF, ET_TO_TOKEN, ET_FROM_TOKEN = 0, 1, 2, 3


# ---- edge sets ------------------------------------------------------------------------------------------------------
def typed_graph_edges(edge_index, num_nodes):
    """Graph edges + exactly one self loop per node, typed 0 (neighbour) / 1 (self)."""
    ei = add_self_loops(edge_index, num_nodes)                      # existing loops dropped, one loop per node appended last
    et = torch.full((ei.shape[1],), ET_NEIGHBOUR, dtype=torch.long, device=ei.device)
    et[ei.shape[1] - num_nodes:] = ET_SELF
    return ei, et


def graphormer_edges(edge_index, num_nodes):
    """``typed_graph_edges`` plus the global token ``T = num_nodes``: (i -> T) type 2, (T -> i) type 3, (T -> T) type 1."""
    ei, et = typed_graph_edges(edge_index, num_nodes)
    tok_ei, to_token = virtual_node_edges(num_nodes, device=ei.device)
    tok_et = torch.where(to_token, ET_TO_TOKEN, ET_FROM_TOKEN)
    loop = torch.full((2, 1), num_nodes, device=ei.device)
    return torch.cat([ei, tok_ei, loop], dim=1), torch.cat([et, tok_et, tok_et.new_tensor([ET_SELF])])


def khop_typed_edges(edge_index, num_nodes, max_two_hop=None, seed=0):
    """2-hop mask with relation type = shortest-path bucket (0 self, 1 neighbour, 2 two hops)."""
    return khop_edges(edge_index, num_nodes, max_two_hop, seed)


def type_local_block(grid, block_edge_index):
    """Types of a local block that already contains the self loops: 1 for self loops, else 0."""
    c_lo, _ = grid.col_block_range()
    row_ids = grid.row_block_ids().to(block_edge_index.device)
    return ((block_edge_index[0] + c_lo) == row_ids[block_edge_index[1]]).long()


def token_edges_local(grid, num_nodes, device):
    """Local edges / types of the global token ``T = num_nodes`` for this rank's block, from the block's ranges only."""
    T = num_nodes
    if grid.n_pad <= num_nodes:
        raise ValueError("the global token needs a padded node slot (n_pad > num_nodes)")
    c_lo, c_hi = grid.col_block_range()
    row_ids = grid.row_block_ids().to(device)
    real_rows = torch.nonzero(row_ids < num_nodes).squeeze(1)
    found = []                                   # (sources, destinations, type) triples in local numbering

    def emit(src, dst, kind):
        src, dst = torch.broadcast_tensors(torch.as_tensor(src, device=device), torch.as_tensor(dst, device=device))
        found.append((src.reshape(-1), dst.reshape(-1), torch.full((src.numel(),), kind, dtype=torch.long, device=device)))
    token_is_my_column = c_lo <= T < c_hi
    token_is_my_row = int(grid.owner_of(torch.tensor([T]))[0][0]) == grid.r
    if token_is_my_column:                       # the token feeds every real row of my row block
        emit(T - c_lo, real_rows, ET_FROM_TOKEN)
    if token_is_my_row:                          # every real column of my column block feeds the token's row
        t_row = int(grid.global_to_row_local(torch.tensor([T]))[0])
        emit(torch.arange(0, max(min(c_hi, num_nodes) - c_lo, 0), device=device), t_row, ET_TO_TOKEN)
        if token_is_my_column:
            emit([T - c_lo], [t_row], ET_SELF)
    if not found:
        none = torch.zeros(0, dtype=torch.long, device=device)
        return torch.stack([none, none]), none
    src, dst, kinds = (torch.cat(part) for part in zip(*found))
    return torch.stack([src, dst]), kinds


def owned_degrees(grid, block_edge_index, block_edge_type, device, neighbour_type=ET_NEIGHBOUR):
    """(in_degree, out_degree) of the owned nodes over the neighbour-typed edges.  In-degrees are counted on the row
    block and summed over the row group; out-degrees on the column block, summed over the column group."""
    sel = block_edge_type == neighbour_type
    indeg = torch.zeros(grid.n_row_block, dtype=torch.float64, device=device)
    indeg.index_add_(0, block_edge_index[1][sel], torch.ones(int(sel.sum()), dtype=torch.float64, device=device))
    outdeg = torch.zeros(grid.n_col_block, dtype=torch.float64, device=device)
    outdeg.index_add_(0, block_edge_index[0][sel], torch.ones(int(sel.sum()), dtype=torch.float64, device=device))
    if group_size(grid.row_group) > 1:
        dist.all_reduce(indeg, group=grid.row_group)
    if group_size(grid.col_group) > 1:
        dist.all_reduce(outdeg, group=grid.col_group)
    if grid.p_heads > 1:                       # the head-group ranks hold the same block: nothing to add
        pass
    return (indeg[grid.row_pos * grid.chunk:(grid.row_pos + 1) * grid.chunk].long(),
            outdeg[grid.col_pos * grid.chunk:(grid.col_pos + 1) * grid.chunk].long())


def owned_in_degree(grid, block_edge_index, block_edge_type, device):
    return owned_degrees(grid, block_edge_index, block_edge_type, device)[0]


def token_owned_row(grid, num_nodes):
    lo, hi = grid.owned_range()
    return num_nodes - lo if lo <= num_nodes < hi else None


# ---- single-process references -----------------------------------------------------------------------------------
def ref_attention(q, k, v, edge_index, etype=None, bias=None, scale=None):
    """Softmax attention over the edges; q on the destination side, k / v on the source side."""
    from ..attention.ref import masked_sparse_attention_ref
    return masked_sparse_attention_ref(q, k, v, edge_index, edge_type=etype, bias=bias, score="biased" if bias is not None else "dot",
                                       norm="softmax", scale=scale)


def _per_head(mod, rows):
    """``(q, k, v)`` of ``rows`` by the module's three projections, each viewed as ``[n, heads, head dim]``."""
    return tuple(proj(rows).view(rows.shape[0], mod.h, mod.d) for proj in (mod.q, mod.k, mod.v))


class UniMPLayerRef(nn.Module):
    def __init__(self, dim, heads, dropout):
        super().__init__()
        self.h, self.d, self.dropout = heads, dim // heads, dropout
        self.q, self.k, self.v, self.r = (nn.Linear(dim, dim) for _ in range(4))
        self.gate = nn.Linear(3 * dim, 1)
        self.ln = K.LayerNorm(dim)

    def combine(self, x, o):
        r = K.linear(x, self.r.weight, self.r.bias)
        return K.gated_residual(r, o.to(r.dtype), self.gate.weight, self.gate.bias, self.ln, self.dropout, self.training)

    def forward(self, x, edge_index):
        return self.combine(x, ref_attention(*_per_head(self, x), edge_index).flatten(1))


class UniMPRef(nn.Module):
    """Label-aware input (a class embedding added where a training label is visible; the padding row means "hidden"),
    ``num_layers`` gated-residual attention layers, linear classifier."""

    def __init__(self, dim_in, dim_hidden, dim_out, num_layers, num_heads, dropout=0.3, num_classes_label=None):
        super().__init__()
        self.pre_lin, self.head, self.dropout = nn.Linear(dim_in, dim_hidden), nn.Linear(dim_hidden, dim_out), dropout
        self.label_emb = None
        if num_classes_label:
            self.label_emb = nn.Embedding(num_classes_label + 1, dim_hidden, padding_idx=num_classes_label)
        self.layers = nn.ModuleList(UniMPLayerRef(dim_hidden, num_heads, dropout) for _ in range(num_layers))

    def inputs(self, x, label_feat=None):
        rows = self.pre_lin(x)
        if label_feat is not None and self.label_emb is not None:
            rows = rows + self.label_emb(label_feat)
        return F.dropout(rows, self.dropout, self.training)

    def forward(self, x, edge_index, label_feat=None):
        rows = self.inputs(x, label_feat)
        for layer in self.layers:
            rows = layer(rows, edge_index)
        return self.head(rows)


class GraphormerBlockRef(nn.Module):
    def __init__(self, dim, ffn, heads, dropout):
        super().__init__()
        self.h, self.d, self.dropout = heads, dim // heads, dropout
        self.ln1 = K.LayerNorm(dim)
        self.q, self.k, self.v, self.o = (nn.Linear(dim, dim) for _ in range(4))
        self.ln2 = K.LayerNorm(dim)
        self.ff1, self.ff2 = nn.Linear(dim, ffn), nn.Linear(ffn, dim)

    def finish(self, x, o):
        """Output projection + residual, then the GELU FFN + residual (owned rows)."""
        x = x + F.dropout(K.linear(o.to(x.dtype), self.o.weight, self.o.bias), self.dropout, self.training)
        y = K.linear(K.linear(self.ln2(x), self.ff1.weight, self.ff1.bias, activation="gelu"), self.ff2.weight, self.ff2.bias)
        return x + F.dropout(y, self.dropout, self.training)

    def forward(self, x, edge_index, etype, attn_bias):
        mixed = ref_attention(*_per_head(self, self.ln1(x)), edge_index, etype, attn_bias)
        return self.finish(x, mixed.flatten(1))


class GraphormerNodeRef(nn.Module):
    """``x`` has one row per (padded) node; ``token_id`` (or ``None``) is the row replaced by the graph token."""

    def __init__(self, dim_in, dim_hidden, dim_out, num_layers, num_heads, dropout=0.3, max_degree=64, ffn_mult=2,
                 num_edge_types=4, out_degree=False):
        super().__init__()
        self.dropout, self.max_degree = dropout, max_degree
        self.pre_lin = nn.Linear(dim_in, dim_hidden)
        self.degree_emb = nn.Embedding(max_degree + 1, dim_hidden)
        self.out_degree_emb = nn.Embedding(max_degree + 1, dim_hidden) if out_degree else None
        self.graph_token = nn.Embedding(1, dim_hidden)
        self.attn_bias = nn.Parameter(torch.zeros(num_edge_types, num_heads))
        self.layers = nn.ModuleList([GraphormerBlockRef(dim_hidden, ffn_mult * dim_hidden, num_heads, dropout) for _ in range(num_layers)])
        self.final_ln = K.LayerNorm(dim_hidden)
        self.head = nn.Linear(dim_hidden, dim_out)

    def embed(self, x, degree, out_degree=None, token_row=None):
        h = K.linear(x, self.pre_lin.weight, self.pre_lin.bias)
        if degree is not None:
            two = self.out_degree_emb is not None and out_degree is not None
            h = K.embed_add(h, self.degree_emb, degree.clamp(max=self.max_degree), self.out_degree_emb if two else None,
                            out_degree.clamp(max=self.max_degree) if two else None)
        elif self.out_degree_emb is not None and out_degree is not None:
            h = K.embed_add(h, self.out_degree_emb, out_degree.clamp(max=self.max_degree))
        if token_row is not None:
            h = torch.cat([h[:token_row], self.graph_token.weight.to(h.dtype), h[token_row + 1:]], dim=0)
        else:
            h = h + 0.0 * self.graph_token.weight.sum().to(h.dtype)       # keeps the parameter in the autograd graph
        return F.dropout(h, self.dropout, self.training)

    def forward(self, x, edge_index, etype, degree, token_id=None, out_degree=None):
        h = self.embed(x, degree, out_degree, token_id)
        for layer in self.layers:
            h = layer(h, edge_index, etype, self.attn_bias)
        return self.head(self.final_ln(h))


# ---- distributed layers ------------------------------------------------------------------------------------------------
class _BlockAttention(nn.Module):
    """Softmax block attention of a model layer: fused-communication form on a 2D grid, head-parallel on a 3D grid.
    ``proj(y_rows, which)`` applies the layer's q / k / v projection."""

    def __init__(self, grid, attn_block, heads, head_dim, backend, score, comm_dtype, rs_dtype):
        super().__init__()
        self.grid, self.h, self.d, self.comm_dtype, self.rs_dtype = grid, heads, head_dim, comm_dtype, rs_dtype
        if grid.p_heads > 1:
            self.op = DistHeadSparseAttention(grid, attn_block, heads, head_dim, backend=backend, score=score, norm="softmax",
                                              comm_dtype=comm_dtype, rs_dtype=rs_dtype)
        else:
            self.op = DistAttentionPartial(grid, attn_block, heads, head_dim, backend=backend, score=score, norm="softmax")

    def forward(self, y, lq, lk, lv, bias=None):
        g, h, d = self.grid, self.h, self.d
        n = y.shape[0]
        if g.p_heads > 1:
            q, k, v = (K.linear(y, l.weight, l.bias).view(n, h, d) for l in (lq, lk, lv))
            return self.op(q, k, v, None, bias).reshape(n, h * d)
        y_col = all_gather_rows(y, g.col_group, self.comm_dtype)
        y_row = all_gather_rows(y, g.row_group, self.comm_dtype)
        q = K.linear(y_row, lq.weight, lq.bias).view(-1, h, d)
        kv = K.linear(y_col, torch.cat([lk.weight, lv.weight], 0), torch.cat([lk.bias, lv.bias], 0))
        k, v = kv[:, :h * d].contiguous().view(-1, h, d), kv[:, h * d:].contiguous().view(-1, h, d)
        acc, l, m = self.op(q, k, v, None, bias)
        o, _ = combine_partials(acc, l, m, g, "softmax", 1e-6, rs_dtype=self.rs_dtype)
        return o.reshape(n, h * d)


class DistUniMPLayerFused(UniMPLayerRef):
    def __init__(self, grid, attn_block, dim, heads, dropout, backend="cuda", comm_dtype=None, rs_dtype=None):
        super().__init__(dim, heads, dropout)
        self.attn = _BlockAttention(grid, attn_block, heads, dim // heads, backend, "dot", comm_dtype, rs_dtype)

    def forward(self, x):
        return self.combine(x, self.attn(x, self.q, self.k, self.v))


class DistGraphormerLayerFused(GraphormerBlockRef):
    def __init__(self, grid, attn_block, dim, ffn, heads, dropout, backend="cuda", comm_dtype=None, rs_dtype=None):
        super().__init__(dim, ffn, heads, dropout)
        self.attn = _BlockAttention(grid, attn_block, heads, dim // heads, backend, "biased", comm_dtype, rs_dtype)

    def forward(self, x, attn_bias):
        return self.finish(x, self.attn(self.ln1(x), self.q, self.k, self.v, attn_bias))


class DistGTVariant(nn.Module):
    """UniMP or Graphormer-node on a 2D or 3D grid; parameter names match the references."""

    def __init__(self, grid, attn_block_ei, attn_block_et, dim_in, dim_hidden, dim_out, num_layers, num_heads, model="unimp",
                 dropout=0.3, backend="cuda", comm_dtype=None, rs_dtype=None, checkpoint=False, num_classes_label=None,
                 max_degree=64, token_row=None, ffn_mult=2, num_edge_types=4, out_degree=False):
        super().__init__()
        if model not in ("unimp", "graphormer"):
            raise ValueError(model)
        self.grid, self.model, self.dropout, self.checkpoint = grid, model, dropout, checkpoint
        self.max_degree, self.token_row = max_degree, token_row
        block = AttentionBlock(grid, attn_block_ei, attn_block_et)
        self.block = block
        if model == "unimp":
            self.pre_lin = nn.Linear(dim_in, dim_hidden)
            self.label_emb = nn.Embedding(num_classes_label + 1, dim_hidden, padding_idx=num_classes_label) if num_classes_label else None
            self.layers = nn.ModuleList([DistUniMPLayerFused(grid, block, dim_hidden, num_heads, dropout, backend, comm_dtype, rs_dtype)
                                         for _ in range(num_layers)])
            self.head = nn.Linear(dim_hidden, dim_out)
        else:
            core = GraphormerNodeRef(dim_in, dim_hidden, dim_out, 0, num_heads, dropout, max_degree, ffn_mult, num_edge_types, out_degree)
            self.pre_lin, self.degree_emb, self.out_degree_emb = core.pre_lin, core.degree_emb, core.out_degree_emb
            self.graph_token, self.attn_bias, self.final_ln, self.head = core.graph_token, core.attn_bias, core.final_ln, core.head
            self._embed = GraphormerNodeRef.embed
            self.label_emb = None
            self.layers = nn.ModuleList([DistGraphormerLayerFused(grid, block, dim_hidden, ffn_mult * dim_hidden, num_heads, dropout,
                                                                  backend, comm_dtype, rs_dtype) for _ in range(num_layers)])

    def load_ref_state_dict(self, sd):
        self.load_state_dict(sd)

    def forward(self, x_loc, label_feat=None, degree_loc=None, out_degree_loc=None):
        if self.model == "unimp":
            h = K.linear(x_loc, self.pre_lin.weight, self.pre_lin.bias)
            if self.label_emb is not None and label_feat is not None:
                h = K.embed_add(h, self.label_emb, label_feat)
            h = F.dropout(h, self.dropout, self.training)
        else:
            h = self._embed(self, x_loc, degree_loc, out_degree_loc, self.token_row)
        for layer in self.layers:
            args = (h, self.attn_bias) if self.model == "graphormer" else (h,)
            if self.checkpoint and self.training:
                h = torch.utils.checkpoint.checkpoint(layer, *args, use_reentrant=False)
            else:
                h = layer(*args)
        if self.model == "graphormer":
            h = self.final_ln(h)
        return K.linear(h, self.head.weight, self.head.bias)

    def structure_bytes(self):
        return self.block.nbytes(set())

    def compaction_stats(self):
        return 0, 0
