"""The global token of an Exphormer attention graph without its row and column in the sparse structure.

A global token (one extra node connected to and from every node, edge type 2; the benchmark graphs have one) puts ``n`` edges into
one row and ``n`` into one column of the attention mask.  On a 2D grid those land on the ranks that hold the token's row block
and column block: every sparse pass of those ranks is longer than everybody else's, and the others wait for them in the next
collective.  Both pieces are dense and tiny, so they need not be edges at all:

* **column** (every node attends to the token): for an owned row ``i`` one more term ``p_i = exp(clamp(scale * (q_i * g_2) . k_t))``
  with the token's key and value, ``acc_i += p_i v_t``, ``l_i += p_i``: element-wise work on the owned rows of every rank;
* **row** (the token attends to every node): ``acc_t = sum_j p_j v_j``, ``l_t = sum_j p_j`` with ``p_j = exp(clamp(scale * (q_t * g_2) . k_j))``:
  every rank reduces over ITS OWNED nodes and one all-reduce of ``H d + H`` numbers completes the sum, which the token's owner
  adds to the token's row.

``DenseToken.add`` does this to the unnormalised ``(acc, l)`` of the owned rows (the partial-softmax state adds, which is why the
clamp-exp weights of the Exphormer layer allow it), with torch operations that autograd differentiates; the token's features travel
to all ranks as a sum in which only the owner's term is non-zero.  Scores against one key (or from one query) are linear in ``x``, so
the owned rows' Q, K and V are never formed: per layer two ``[O, d] x [d, H]`` products, one ``[H, O] x [O, d]`` product and one update
of ``acc`` beside the block projections of the sparse path.  The sparse structure is then built without the token's
edges (``exphormer_workload(token_dense=True)``, ``train_dist --token_dense``).

Every rank must run the same collectives in forward and backward, so every term is tied to ``x`` on every rank (with a zero factor
where the rank contributes nothing): a rank whose part of the graph were cut off from ``x`` would skip a backward collective.

The reference has no counterpart: its training graphs carry no global token (``gt3d/gt3d/train/train_dist.py:427-428,471-476``); only
its kernel benchmarks do (``gt3d/bench/bench_attention_single_gpu.py:89-97``), as edges.
"""
import torch

from .collectives import all_reduce_sum


class DenseToken:
    def __init__(self, grid, token_node):
        lo, hi = grid.owned_range()
        self.node = int(token_node)
        self.row = self.node - lo if lo <= self.node < hi else None
        rows = torch.arange(lo, hi)
        self.others = ((rows < grid.num_nodes) & (rows != self.node)).float()       # owned real nodes other than the token
        self.onehot = (rows == self.node).float()

    def _to(self, x):
        if self.others.device != x.device:
            self.others, self.onehot = self.others.to(x.device), self.onehot.to(x.device)

    @staticmethod
    def _pad8(v):
        pad = (-v.numel()) % 8
        return torch.cat([v, v.new_zeros(pad)]) if pad else v

    def add(self, layer, x, gate, acc, l):
        """``(acc, l)`` of the owned rows (fp32, unnormalised, any of ``[O, H d]`` / ``[O, H, d]``) plus the token's row and column."""
        self._to(x)
        o, h, d = x.shape[0], layer.num_heads, layer.d_head
        hd = h * d
        scale, (c_lo, c_hi) = float(layer.attn.scale), layer.attn.clamp
        ct = torch.float64 if x.dtype == torch.float64 else torch.float32     # arithmetic of the dense terms
        g2 = gate[2].to(ct).reshape(h, d)
        shape = acc.shape
        acc, l = acc.to(ct).reshape(o, h, d), l.to(ct).reshape(o, h)
        onehot, mask = self.onehot.to(ct), self.others.to(ct).unsqueeze(1)
        # the token's features on every rank: a sum over ranks in which only the owner's term is non-zero
        x_t = all_reduce_sum(self._pad8((x.to(ct) * onehot.unsqueeze(1)).sum(0)))[:x.shape[1]]
        din = x.shape[1]
        wq, wk, wv = (w.weight.to(ct).view(h, d, din) for w in (layer.q, layer.k, layer.v))
        q_t, k_t, v_t = (torch.einsum("hdi,i->hd", w, x_t) for w in (wq, wk, wv))
        xc = x.to(ct)
        # Scores against ONE key (or from ONE query) are linear in x: s_i[h] = x_i . u[h] with u[h] = scale * W_q[h]^T (g_2[h] * k_t[h]), so
        # the owned rows' Q, K and V are never formed: two [O, d_in] x [d_in, H] products and one [H, O] x [O, d_in] product replace
        # three [O, d_in] x [d_in, H d] projections, and every element-wise pass below runs on [O, H].
        u_col = torch.einsum("hd,hdi->hi", g2 * k_t, wq) * scale
        p_col = torch.exp((xc @ u_col.t()).clamp(c_lo, c_hi)) * mask                 # column of the token: one more source per owned row
        acc = acc + p_col.unsqueeze(-1) * v_t
        l = l + p_col
        u_row = torch.einsum("hd,hdi->hi", g2 * q_t, wk) * scale
        p_row = torch.exp((xc @ u_row.t()).clamp(c_lo, c_hi)) * mask                 # row of the token: weights of the owned nodes
        z = p_row.t() @ xc                                                           # [H, d_in]: sum_j p_j x_j per head
        part = torch.cat([torch.einsum("hi,hdi->hd", z, wv).reshape(-1), p_row.sum(0)])
        tot = all_reduce_sum(self._pad8(part))
        acc = acc + onehot.view(o, 1, 1) * tot[:hd].view(1, h, d)
        l = l + onehot.view(o, 1) * tot[hd:hd + h].view(1, h)
        return acc.reshape(shape), l
