"""TorchGT-style node-level Graphormer on the block attention operator, for same-model / same-batch comparisons with
TorchGT: pre-LayerNorm blocks, dot-product scores with the clamp(-5, 5)-exp normalisation (no edge gate), mask = the 1-hop
edges of the batch sub-graph plus a global token that is node 0 (model definition: reference
``gt3d/gt3d/models/graphormer_node.py:16-131``; parameter names are kept, so state dicts are interchangeable).

One layer class serves every placement.  Its dense halves (``project``: LayerNorm-ed rows to Q / K / V with the K | V, or
Q | K | V, weights stacked into ONE GEMM; ``close``: output projection, residual, FFN with the GELU fused into the first
GEMM's epilogue) are shared; where the rows come from and how the attention output returns is the layer's ``route``:

  ``local``   one device: all rows are here;
  ``plain``   2D grid: the distributed operator gathers / reduce-scatters inside (``DistMaskedSparseAttention``);
  ``fused``   2D grid: LN(x) is gathered once per group, projected on the gathered rows, the unnormalised partials are
              merged by one reduce-scatter (``DistAttentionPartial`` + ``combine_partials``).
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..attention import BlockCSR
from ..ops import functional as K
from ..parallel.attention import AttentionBlock, DistAttentionPartial, DistMaskedSparseAttention, combine_partials
from ..parallel.collectives import all_gather_rows


def _stacked(*linears):
    """Weights and biases of several ``nn.Linear`` stacked along the output axis (one GEMM instead of several)."""
    return torch.cat([m.weight for m in linears], 0), torch.cat([m.bias for m in linears], 0)


class _Layer(nn.Module):
    def __init__(self, hidden, ffn, heads, dropout, route, operator, grid=None, comm_dtype=None, rs_dtype=None):
        super().__init__()
        if route not in ("local", "plain", "fused"):
            raise ValueError(route)
        self.heads, self.head_dim, self.p = heads, hidden // heads, dropout
        self.route, self.operator = route, operator               # operator: callable(q, k, v) on [rows, H, d_head] tensors
        self.grid, self.comm_dtype, self.rs_dtype = grid, comm_dtype, rs_dtype
        for name in ("q", "k", "v", "o"):
            setattr(self, name, nn.Linear(hidden, hidden))
        self.ln1, self.ln2 = K.LayerNorm(hidden), K.LayerNorm(hidden)
        self.ff1, self.ff2 = nn.Linear(hidden, ffn), nn.Linear(ffn, hidden)

    def _heads(self, t):
        return t.view(t.shape[0], self.heads, self.head_dim)

    def project(self, rows_q, rows_kv):
        width = self.heads * self.head_dim
        if rows_q is rows_kv:
            w, b = _stacked(self.q, self.k, self.v)
            q, k, v = K.split_columns(K.linear(rows_q, w, b), [width] * 3)
        else:
            q = K.linear(rows_q, self.q.weight, self.q.bias)
            w, b = _stacked(self.k, self.v)
            k, v = K.split_columns(K.linear(rows_kv, w, b), [width] * 2)
        return self._heads(q), self._heads(k), self._heads(v)

    def close(self, x, mixed):
        x = x + F.dropout(K.linear(mixed.to(x.dtype), self.o.weight, self.o.bias), self.p, self.training)
        hidden = K.linear(self.ln2(x), self.ff1.weight, self.ff1.bias, activation="gelu")
        return x + F.dropout(K.linear(hidden, self.ff2.weight, self.ff2.bias), self.p, self.training)

    def forward(self, x):
        y = self.ln1(x)
        if self.route == "fused":
            g = self.grid
            q, k, v = self.project(all_gather_rows(y, g.row_group, self.comm_dtype), all_gather_rows(y, g.col_group, self.comm_dtype))
            mixed, _ = combine_partials(*self.operator(q, k, v), g, "clampexp", 1e-6, rs_dtype=self.rs_dtype)
        else:
            mixed = self.operator(*self.project(y, y))
        return self.close(x, mixed.reshape(x.shape[0], -1))


class _Stack(nn.Module):
    """Encoder, graph token, layers, final norm and classifier shared by both models."""

    def _build(self, dim_in, hidden, num_classes, input_dropout, layers):
        self.encoder = nn.Linear(dim_in, hidden)
        self.graph_token = nn.Embedding(1, hidden)
        self.input_dropout = input_dropout
        self.layers = nn.ModuleList(layers)
        self.final_ln = K.LayerNorm(hidden)
        self.out = nn.Linear(hidden, num_classes)

    def _run(self, h):
        h = F.dropout(h, self.input_dropout, self.training)
        for layer in self.layers:
            h = layer(h)
        return self.final_ln(h)

    def _embed(self, x):
        return K.linear(x, self.encoder.weight, self.encoder.bias)

    def _classify(self, h):
        return K.linear(h, self.out.weight, self.out.bias)


class GraphormerNode(_Stack):
    """Single device.  ``edge_index`` is over the batch nodes with node 0 = the global token (TorchGT layout); ``x`` holds the
    features of nodes ``1 .. n``, the token's row is a learned embedding."""

    def __init__(self, dim_in, hidden, ffn, heads, layers, num_classes, edge_index, num_nodes, dropout=0.3, input_dropout=0.1,
                 backend="cuda"):
        super().__init__()
        self.csr = BlockCSR.from_edges(edge_index, num_nodes, num_nodes)
        self.backend = backend
        self._build(dim_in, hidden, num_classes, input_dropout,
                    [_Layer(hidden, ffn, heads, dropout, "local", self._attend) for _ in range(layers)])

    def _attend(self, q, k, v):
        if self.backend == "cuda":
            from ..attention.backend_cuda import masked_sparse_attention_cuda as op
        else:
            from ..attention.backend_torch import masked_sparse_attention_torch as op
        self.csr = self.csr.to(q.device)
        return op(q, k, v, self.csr, score="dot", norm="clampexp")

    def forward(self, x):
        rows = torch.cat([self.graph_token.weight.to(x.dtype), self._embed(x)], dim=0)
        return self._classify(self._run(rows)[1:])


class DistGraphormerNode(_Stack):
    """2D-distributed: the global token is node 0 of the padded id space (owned by the rank whose chunk starts at 0).
    ``forward`` takes and returns this rank's chunk of rows."""

    def __init__(self, grid, attn_block, dim_in, hidden, ffn, heads, layers, num_classes, dropout=0.3, input_dropout=0.1,
                 backend="cuda", comm_dtype=None, fused=False, rs_dtype=None):
        super().__init__()
        self.grid = grid
        if not isinstance(attn_block, AttentionBlock):
            attn_block = AttentionBlock(grid, *attn_block)
        opts = dict(backend=backend, score="dot", norm="clampexp")
        if fused:
            ops = [DistAttentionPartial(grid, attn_block, heads, hidden // heads, **opts) for _ in range(layers)]
            stack = [_Layer(hidden, ffn, heads, dropout, "fused", op, grid, comm_dtype, rs_dtype) for op in ops]
        else:
            ops = [DistMaskedSparseAttention(grid, attn_block, heads, hidden // heads, comm_dtype=comm_dtype, **opts) for _ in range(layers)]
            stack = [_Layer(hidden, ffn, heads, dropout, "plain", op) for op in ops]
        self.attns = nn.ModuleList(ops)
        self._build(dim_in, hidden, num_classes, input_dropout, stack)

    def forward(self, x_loc):
        rows = self._embed(x_loc)
        token = self.graph_token.weight.to(rows.dtype)
        if self.grid.owned_range()[0] == 0:
            rows = torch.cat([token, rows[1:]], dim=0)
        else:
            rows = rows + 0.0 * token.sum()            # every rank touches the token so that its gradient exists everywhere
        return self._classify(self._run(rows))
