"""TorchGT-style node-level Graphormer on the block attention operator: pre-LayerNorm blocks, dot-product scores with
the clamp(-5, 5)-exp normalisation (no edge gate), mask = 1-hop edges of the batch sub-graph plus a global token that
is node 0.  Used for same-model / same-batch comparisons with TorchGT (reference:
``gt3d/gt3d/models/graphormer_node.py:16-131``).  ``GraphormerNode`` is the single-device model, ``DistGraphormerNode``
the 2D-distributed one (plain or fused communication)."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..attention import BlockCSR
from ..ops import functional as K
from ..parallel.attention import AttentionBlock, DistAttentionPartial, DistMaskedSparseAttention, combine_partials
from ..parallel.collectives import all_gather_rows


class _Block(nn.Module):
    def __init__(self, hidden, ffn, heads, dropout, attention):
        super().__init__()
        self.h, self.dh, self.dropout = heads, hidden // heads, dropout
        self.ln1 = K.LayerNorm(hidden)
        self.q, self.k, self.v, self.o = (nn.Linear(hidden, hidden) for _ in range(4))
        self.ln2 = K.LayerNorm(hidden)
        self.ff1, self.ff2 = nn.Linear(hidden, ffn), nn.Linear(ffn, hidden)
        self.attention = attention                     # callable(q, k, v) -> o, all [n, H, dh]

    def _finish(self, x, o):
        x = x + F.dropout(K.linear(o.to(x.dtype), self.o.weight, self.o.bias), self.dropout, self.training)
        y = K.linear(K.linear(self.ln2(x), self.ff1.weight, self.ff1.bias, activation="gelu"), self.ff2.weight, self.ff2.bias)
        return x + F.dropout(y, self.dropout, self.training)

    def forward(self, x):
        n = x.shape[0]
        y = self.ln1(x)
        q, k, v = (K.linear(y, l.weight, l.bias).view(n, self.h, self.dh) for l in (self.q, self.k, self.v))
        return self._finish(x, self.attention(q, k, v).reshape(n, -1))


class _FusedDistBlock(_Block):
    """Fused communication on the 2D grid: the LayerNorm-ed input is gathered once per block, projected locally, the
    partials are merged by one reduce-scatter."""

    def __init__(self, hidden, ffn, heads, dropout, attn_partial, grid, comm_dtype=None, rs_dtype=None):
        super().__init__(hidden, ffn, heads, dropout, attn_partial)
        self.grid, self.comm_dtype, self.rs_dtype = grid, comm_dtype, rs_dtype

    def forward(self, x):
        g, n = self.grid, x.shape[0]
        y = self.ln1(x)
        y_col = all_gather_rows(y, g.col_group, self.comm_dtype)
        y_row = all_gather_rows(y, g.row_group, self.comm_dtype)
        q = K.linear(y_row, self.q.weight, self.q.bias).view(-1, self.h, self.dh)
        k = K.linear(y_col, self.k.weight, self.k.bias).view(-1, self.h, self.dh)
        v = K.linear(y_col, self.v.weight, self.v.bias).view(-1, self.h, self.dh)
        acc, l, m = self.attention(q, k, v)
        o, _ = combine_partials(acc, l, m, g, "clampexp", 1e-6, rs_dtype=self.rs_dtype)
        return self._finish(x, o.reshape(n, -1))


class GraphormerNode(nn.Module):
    """Single device.  ``edge_index`` is over the batch nodes with node 0 = the global token (TorchGT layout)."""

    def __init__(self, dim_in, hidden, ffn, heads, layers, num_classes, edge_index, num_nodes, dropout=0.3, input_dropout=0.1,
                 backend="cuda"):
        super().__init__()
        self.encoder = nn.Linear(dim_in, hidden)
        self.graph_token = nn.Embedding(1, hidden)
        self.input_dropout = input_dropout
        self.csr = BlockCSR.from_edges(edge_index, num_nodes, num_nodes)
        self.backend = backend

        def attention(q, k, v):
            if self.backend == "cuda":
                from ..attention.backend_cuda import masked_sparse_attention_cuda as fn
            else:
                from ..attention.backend_torch import masked_sparse_attention_torch as fn
            self.csr = self.csr.to(q.device)
            return fn(q, k, v, self.csr, score="dot", norm="clampexp")
        self.layers = nn.ModuleList([_Block(hidden, ffn, heads, dropout, attention) for _ in range(layers)])
        self.final_ln = K.LayerNorm(hidden)
        self.out = nn.Linear(hidden, num_classes)

    def forward(self, x):
        h = torch.cat([self.graph_token.weight.to(x.dtype), K.linear(x, self.encoder.weight, self.encoder.bias)], dim=0)
        h = F.dropout(h, self.input_dropout, self.training)
        for layer in self.layers:
            h = layer(h)
        return K.linear(self.final_ln(h)[1:], self.out.weight, self.out.bias)


class DistGraphormerNode(nn.Module):
    """2D-distributed: the global token is node 0 of the padded id space (owned by the rank whose chunk starts at 0)."""

    def __init__(self, grid, attn_block, dim_in, hidden, ffn, heads, layers, num_classes, dropout=0.3, input_dropout=0.1,
                 backend="cuda", comm_dtype=None, fused=False, rs_dtype=None):
        super().__init__()
        self.grid = grid
        self.encoder = nn.Linear(dim_in, hidden)
        self.graph_token = nn.Embedding(1, hidden)
        self.input_dropout = input_dropout
        if not isinstance(attn_block, AttentionBlock):
            attn_block = AttentionBlock(grid, *attn_block)
        if fused:
            self.attns = nn.ModuleList([DistAttentionPartial(grid, attn_block, heads, hidden // heads, backend=backend, score="dot",
                                                             norm="clampexp") for _ in range(layers)])
            self.layers = nn.ModuleList([_FusedDistBlock(hidden, ffn, heads, dropout, a, grid, comm_dtype, rs_dtype) for a in self.attns])
        else:
            self.attns = nn.ModuleList([DistMaskedSparseAttention(grid, attn_block, heads, hidden // heads, backend=backend, score="dot",
                                                                  norm="clampexp", comm_dtype=comm_dtype) for _ in range(layers)])
            self.layers = nn.ModuleList([_Block(hidden, ffn, heads, dropout, a) for a in self.attns])
        self.final_ln = K.LayerNorm(hidden)
        self.out = nn.Linear(hidden, num_classes)

    def forward(self, x_loc):
        h = K.linear(x_loc, self.encoder.weight, self.encoder.bias)
        if self.grid.owned_range()[0] == 0:
            h = torch.cat([self.graph_token.weight.to(h.dtype), h[1:]], dim=0)
        else:
            h = h + 0.0 * self.graph_token.weight.sum().to(h.dtype)
        h = F.dropout(h, self.input_dropout, self.training)
        for layer in self.layers:
            h = layer(h)
        return K.linear(self.final_ln(h), self.out.weight, self.out.bias)
