"""Single-GPU / single-process Exphormer with a selectable attention back-end (``ref`` edge list, ``torch`` CSR,
``cuda`` sm_100a kernels); parameters and mathematics of :class:`ExphormerRef`, so checkpoints are interchangeable
(reference: ``gt3d/gt3d/models/exphormer.py:20-82``)."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..attention import BlockCSR, masked_sparse_attention_ref
from ..attention.backend_torch import masked_sparse_attention_torch
from ..ops.sparse import spmm
from .exphormer_ref import ExphormerLayerRef, ExphormerRef, gcn_norm


class AttentionGraph:
    """Attention edge set (graph + expander [+ token] edges) with its CSR, and the normalised GCN matrix, built once."""

    def __init__(self, edge_index, exp_edge_index, num_nodes, token_edge_index=None, dtype=torch.float32):
        self.num_nodes = num_nodes
        self.edge_index, self.etype = ExphormerRef.build_attention_edges(edge_index, exp_edge_index, token_edge_index)
        self.csr = BlockCSR.from_edges(self.edge_index, num_nodes, num_nodes, self.etype)
        ei, w = gcn_norm(edge_index, num_nodes, torch.float64)
        wdt = torch.float32 if dtype in (torch.bfloat16, torch.float16) else dtype
        self.gcn = BlockCSR.from_edges(ei, num_nodes, num_nodes, weight=w.to(wdt))
        self.gcn_edge_index = edge_index

    def to(self, device):
        self.csr, self.gcn = self.csr.to(device), self.gcn.to(device)
        self.edge_index, self.etype = self.edge_index.to(device), self.etype.to(device)
        return self


def _attend(backend, q, k, v, graph, gate):
    """Gated clamp-exp attention over the graph's attention edges on the chosen back-end."""
    opts = dict(gate=gate, score="gated", norm="clampexp")
    if backend == "ref":
        return masked_sparse_attention_ref(q, k, v, graph.edge_index, edge_type=graph.etype, **opts)
    if backend == "torch":
        return masked_sparse_attention_torch(q, k, v, graph.csr, **opts)
    from ..attention.backend_cuda import masked_sparse_attention_cuda
    return masked_sparse_attention_cuda(q, k, v, graph.csr, **opts)


class ExphormerLayer(ExphormerLayerRef):
    """The reference layer's parameters; the bias-free projections that read ``x`` (Q, K, V and the GCN message) run as ONE
    GEMM on the stacked weights, each branch ends in its own residual + norm, then the FFN."""

    def __init__(self, *args, backend="cuda", **kwargs):
        super().__init__(*args, **kwargs)
        self.backend = backend

    def _projected(self, x):
        mats = ([self.q.weight, self.k.weight, self.v.weight] if self.with_attn else []) + ([self.gcn.lin.weight] if self.with_gcn else [])
        out = F.linear(x, torch.cat(mats, 0) if len(mats) > 1 else mats[0])
        return out.split(x.shape[1], dim=1)

    def forward(self, x, graph: AttentionGraph, edge_type_emb):
        rows, heads = x.shape[0], (self.num_heads, self.d_head)
        pieces = list(self._projected(x))
        branch_sum = None
        if self.with_attn:
            q, k, v = (pieces.pop(0).reshape(rows, *heads) for _ in range(3))
            o = _attend(self.backend, q, k, v, graph, self.e(edge_type_emb).view(-1, *heads))
            branch_sum = self.bn_attn(x + F.dropout(o.reshape(rows, -1).to(x.dtype), self.dropout, self.training))
        if self.with_gcn:
            agg = spmm(graph.gcn, pieces.pop(0).contiguous()) + self.gcn.bias
            local = self.bn_local(x + F.dropout(agg, self.dropout, self.training))
            branch_sum = local if branch_sum is None else branch_sum + local
        ffn = F.dropout(F.relu(self.ff1(branch_sum)), self.dropout, self.training)
        return self.bn_ff(branch_sum + F.dropout(self.ff2(ffn), self.dropout, self.training))


class Exphormer(ExphormerRef):
    def __init__(self, dim_in, dim_hidden, dim_out, num_layers, num_heads, dropout=0.3, gnn_dropout=0.3, num_edge_types=2,
                 bn_eps=1e-5, bn_momentum=0.1, backend="cuda", pre_l2norm=True, with_gcn=True, with_attn=True, norm="bn"):
        super().__init__(dim_in, dim_hidden, dim_out, num_layers, num_heads, dropout, gnn_dropout, num_edge_types, bn_eps,
                         bn_momentum, pre_l2norm, with_gcn, with_attn, norm)
        self.layers = nn.ModuleList([ExphormerLayer(dim_hidden, num_heads, dropout, bn_eps, bn_momentum, with_gcn,
                                                    with_attn, norm, backend=backend) for _ in range(num_layers)])

    def forward(self, x, graph: AttentionGraph):
        h = self.pre_mp(x)
        for layer in self.layers:
            h = layer(h, graph, self.edge_type_emb.weight)
        return self.head(h)
