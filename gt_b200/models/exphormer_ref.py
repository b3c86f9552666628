"""Single-process Exphormer ("GCN + Exphormer" GraphGPS MultiModel) written on the edge-list specification.

This is the numerical oracle of the distributed models and the owner of the checkpoint key names:

    edge_type_emb.weight, pre_lin.weight, pre_bn.*, head.{weight,bias},
    layers.{i}.{gcn.lin.weight, gcn.bias, bn_local.*, q.weight, k.weight, v.weight, e.weight, bn_attn.*,
                ff1.{weight,bias}, ff2.{weight,bias}, bn_ff.*}

(the names of the reference's ``ExphormerRef``, ``gt3d/gt3d/models/exphormer_ref.py:69-135``; keys of the official
graphgps checkpoint map onto them through ``official_to_ref_key``, ``:170-205``).

Per layer:  h_local = N(x + Drop(GCN(x)));  h_attn = N(x + Drop(Attn(x)));  h = h_local + h_attn;
            out = N(h + Drop(W2 Drop(ReLU(W1 h)))),   N = BatchNorm (default), LayerNorm or RMSNorm.
Attn: gated scores ``s_ij = sum_f q_if k_jf g[t_ij, f] / sqrt(d_h)`` with ``g = E(edge_type_emb)``, clamp-exp
normalisation, no output projection.  Pre-MP: Linear(no bias) -> N -> Dropout -> ReLU -> L2 normalise.
"""
import re

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..attention.ref import masked_sparse_attention_ref, segment_sum


def gcn_edges_with_self_loops(edge_index, num_nodes):
    """Drop existing self loops and add exactly one per node (PyG ``add_remaining_self_loops``)."""
    keep = edge_index[0] != edge_index[1]
    loops = torch.arange(num_nodes, device=edge_index.device)
    return torch.cat([edge_index[:, keep], torch.stack([loops, loops])], dim=1)


def gcn_norm(edge_index, num_nodes, dtype):
    """``(edge_index with self loops, weights d_dst^-1/2 d_src^-1/2)`` with the in-degree counted on destinations."""
    ei = gcn_edges_with_self_loops(edge_index, num_nodes)
    ones = torch.ones(ei.shape[1], dtype=dtype, device=ei.device)
    deg = segment_sum(ones, ei[1], num_nodes)
    dis = torch.where(deg > 0, deg.pow(-0.5), torch.zeros_like(deg))
    return ei, dis[ei[0]] * dis[ei[1]]


class RMSNorm(nn.Module):
    """Per-node root-mean-square normalisation with a learned scale (no collective)."""

    def __init__(self, dim, eps=1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.to(x.dtype)


def make_norm_ref(kind, dim, eps, momentum):
    if kind == "bn":
        return nn.BatchNorm1d(dim, eps=eps, momentum=momentum)
    if kind == "ln":
        return nn.LayerNorm(dim, eps=eps)
    if kind == "rms":
        return RMSNorm(dim, eps=eps)
    raise ValueError(kind)


class GCNConvRef(nn.Module):
    def __init__(self, dim_in, dim_out):
        super().__init__()
        self.lin = nn.Linear(dim_in, dim_out, bias=False)
        self.bias = nn.Parameter(torch.zeros(dim_out))

    def forward(self, x, edge_index):
        ei, w = gcn_norm(edge_index, x.shape[0], x.dtype)
        return segment_sum(self.lin(x)[ei[0]] * w.unsqueeze(-1), ei[1], x.shape[0]) + self.bias


class ExphormerLayerRef(nn.Module):
    def __init__(self, dim_h, num_heads, dropout, bn_eps=1e-5, bn_momentum=0.1, with_gcn=True, with_attn=True, norm="bn"):
        super().__init__()
        if dim_h % num_heads:
            raise ValueError("hidden size must be divisible by the number of heads")
        self.dim_h, self.num_heads, self.d_head, self.dropout = dim_h, num_heads, dim_h // num_heads, dropout
        self.with_gcn, self.with_attn = with_gcn, with_attn
        if with_gcn:
            self.gcn = GCNConvRef(dim_h, dim_h)
            self.bn_local = make_norm_ref(norm, dim_h, bn_eps, bn_momentum)
        if with_attn:
            self.q, self.k, self.v, self.e = (nn.Linear(dim_h, dim_h, bias=False) for _ in range(4))
            self.bn_attn = make_norm_ref(norm, dim_h, bn_eps, bn_momentum)
        self.ff1 = nn.Linear(dim_h, 2 * dim_h)
        self.ff2 = nn.Linear(2 * dim_h, dim_h)
        self.bn_ff = make_norm_ref(norm, dim_h, bn_eps, bn_momentum)

    def attention(self, x, attn_edge_index, edge_type, edge_type_emb):
        n, h, d = x.shape[0], self.num_heads, self.d_head
        gate = self.e(edge_type_emb).view(-1, h, d)
        o = masked_sparse_attention_ref(self.q(x).view(n, h, d), self.k(x).view(n, h, d), self.v(x).view(n, h, d),
                                        attn_edge_index, edge_type=edge_type, gate=gate, score="gated", norm="clampexp")
        return o.reshape(n, h * d)

    def forward(self, x, edge_index, attn_edge_index, edge_type, edge_type_emb):
        drop = lambda t: F.dropout(t, self.dropout, self.training)                 # noqa: E731
        parts = []
        if self.with_attn:
            parts.append(self.bn_attn(x + drop(self.attention(x, attn_edge_index, edge_type, edge_type_emb))))
        if self.with_gcn:
            parts.append(self.bn_local(x + drop(self.gcn(x, edge_index))))
        h = parts[0] if len(parts) == 1 else parts[0] + parts[1]
        return self.bn_ff(h + drop(self.ff2(drop(F.relu(self.ff1(h))))))


class ExphormerRef(nn.Module):
    def __init__(self, dim_in, dim_hidden, dim_out, num_layers, num_heads, dropout=0.3, gnn_dropout=0.3, num_edge_types=2,
                 bn_eps=1e-5, bn_momentum=0.1, pre_l2norm=True, with_gcn=True, with_attn=True, norm="bn"):
        super().__init__()
        self.gnn_dropout, self.pre_l2norm = gnn_dropout, pre_l2norm
        self.edge_type_emb = nn.Embedding(num_edge_types, dim_hidden)
        self.pre_lin = nn.Linear(dim_in, dim_hidden, bias=False)
        self.pre_bn = make_norm_ref(norm, dim_hidden, bn_eps, bn_momentum)
        self.layers = nn.ModuleList([ExphormerLayerRef(dim_hidden, num_heads, dropout, bn_eps, bn_momentum, with_gcn,
                                                       with_attn, norm) for _ in range(num_layers)])
        self.head = nn.Linear(dim_hidden, dim_out)

    @staticmethod
    def build_attention_edges(edge_index, exp_edge_index, token_edge_index=None):
        """Attention mask = graph edges (type 0) + expander edges (type 1) [+ global-token edges (type 2)]."""
        parts, types = [edge_index, exp_edge_index], [0, 1]
        if token_edge_index is not None:
            parts.append(token_edge_index)
            types.append(2)
        ei = torch.cat(parts, dim=1)
        et = torch.cat([torch.full((p.shape[1],), t, dtype=torch.long, device=ei.device) for p, t in zip(parts, types)])
        return ei, et

    def pre_mp(self, x):
        h = F.relu(F.dropout(self.pre_bn(self.pre_lin(x)), self.gnn_dropout, self.training))
        return F.normalize(h, p=2, dim=1) if self.pre_l2norm else h

    def forward(self, x, edge_index, exp_edge_index, token_edge_index=None):
        attn_ei, et = self.build_attention_edges(edge_index, exp_edge_index, token_edge_index)
        h = self.pre_mp(x)
        for layer in self.layers:
            h = layer(h, edge_index, attn_ei, et, self.edge_type_emb.weight)
        return self.head(h)


# ---- official graphgps checkpoint keys ---------------------------------------------------------------------------
_LAYER_KEYS = {
    "models.0.local_model.lin.weight": "gcn.lin.weight", "models.0.local_model.bias": "gcn.bias",
    "models.1.self_attn.Q.weight": "q.weight", "models.1.self_attn.K.weight": "k.weight",
    "models.1.self_attn.V.weight": "v.weight", "models.1.self_attn.E.weight": "e.weight",
    "ff_linear1.weight": "ff1.weight", "ff_linear1.bias": "ff1.bias", "ff_linear2.weight": "ff2.weight", "ff_linear2.bias": "ff2.bias",
}
_NORM_PREFIX = {"models.0.norm1_local.": "bn_local.", "models.1.norm1_attn.": "bn_attn.", "norm2.": "bn_ff."}
_NORM_FIELDS = ("weight", "bias", "running_mean", "running_var", "num_batches_tracked")


def official_to_ref_key(key: str):
    """Key of this package's state dict for one key of the official graphgps ``MultiModel`` (``None`` if unmapped).
    Edge-type embedding rows are returned as ``'edge_type_emb.weight[i]'``."""
    fixed = {"encoder.edge_encoder.encoder.weight": "edge_type_emb.weight[0]",
             "encoder.exp_edge_fixer.exp_edge_attr.weight": "edge_type_emb.weight[1]",
             "pre_mp.Layer_0.layer.model.weight": "pre_lin.weight"}
    if key in fixed:
        return fixed[key]
    m = re.fullmatch(r"pre_mp\.Layer_0\.post_layer\.0\.(\w+)", key)
    if m:
        return f"pre_bn.{m.group(1)}"
    m = re.fullmatch(r"post_mp\.layer_post_mp\.model\.0\.model\.(weight|bias)", key)
    if m:
        return f"head.{m.group(1)}"
    m = re.fullmatch(r"layers\.(\d+)\.(.+)", key)
    if m:
        idx, rest = m.groups()
        if rest in _LAYER_KEYS:
            return f"layers.{idx}.{_LAYER_KEYS[rest]}"
        for pre, tgt in _NORM_PREFIX.items():
            if rest.startswith(pre) and rest[len(pre):] in _NORM_FIELDS:
                return f"layers.{idx}.{tgt}{rest[len(pre):]}"
    return None


@torch.no_grad()
def load_official_state_dict(model: nn.Module, official_sd: dict, strict: bool = True):
    """Fill ``model`` (any model using the key names above) from an official graphgps state dict."""
    sd = model.state_dict()
    filled = set()
    for key, val in official_sd.items():
        tgt = official_to_ref_key(key)
        if tgt is None:
            if strict:
                raise KeyError(f"unmapped official key {key}")
            continue
        m = re.fullmatch(r"(.+)\[(\d+)\]", tgt)
        if m:
            sd[m.group(1)][int(m.group(2))].copy_(val.reshape(-1))
            filled.add(m.group(1))
        else:
            sd[tgt].copy_(val)
            filled.add(tgt)
    missing = set(sd) - filled
    if strict and missing:
        raise KeyError(f"keys not filled: {sorted(missing)}")
    model.load_state_dict(sd)
    return model
