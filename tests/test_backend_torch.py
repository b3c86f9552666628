"""CSR torch backend vs the edge-list specification (fp64): every score x norm, chunked or not, empty rows, hub."""
import itertools

import pytest
import torch

from gt_b200.attention import BlockCSR, masked_sparse_attention_ref
from gt_b200.attention import backend_torch as bt
from helpers import random_graph


@pytest.mark.parametrize("score,norm,chunk", list(itertools.product(["dot", "gated", "biased"], ["softmax", "clampexp"], [0, 97])))
def test_matches_reference(score, norm, chunk):
    torch.manual_seed(1)
    n, h, d, t = 60, 3, 8, 3
    ei, et = random_graph(n, 4, seed=2)
    blk = BlockCSR.from_edges(ei, n, n, et)
    mk = lambda *s: torch.randn(*s, dtype=torch.float64, requires_grad=True)     # noqa: E731
    q, k, v, gate, bias = mk(n, h, d), mk(n, h, d), mk(n, h, d), mk(t, h, d), mk(t, h)
    kw = dict(score=score, norm=norm, gate=gate if score == "gated" else None, bias=bias if score == "biased" else None)
    o_ref = masked_sparse_attention_ref(q * 3, k, v, ei, edge_type=et, **kw)
    w = torch.randn_like(o_ref)
    g_ref = torch.autograd.grad((o_ref * w).sum(), [t_ for t_ in (q, k, v, gate, bias) if t_ is not None and
                                                    (t_ is not gate or score == "gated") and (t_ is not bias or score == "biased")])
    o = bt.masked_sparse_attention_torch(q * 3, k, v, blk, chunk_edges=chunk, **kw)
    g = torch.autograd.grad((o * w).sum(), [t_ for t_ in (q, k, v, gate, bias) if t_ is not None and
                                            (t_ is not gate or score == "gated") and (t_ is not bias or score == "biased")])
    assert (o - o_ref).abs().max() < 1e-12
    assert o[3].abs().max() == 0 and o[7].abs().max() == 0
    for a, b in zip(g, g_ref):
        assert (a - b).abs().max() < 1e-11


@pytest.mark.parametrize("norm", ["softmax", "clampexp"])
def test_partial_backward_is_gradient_of_partials(norm):
    torch.manual_seed(0)
    n, h, d = 40, 2, 4
    ei, et = random_graph(n, 3, seed=5)
    blk = BlockCSR.from_edges(ei, n, n, et)
    q, k, v = (torch.randn(n, h, d, dtype=torch.float64, requires_grad=True) for _ in range(3))
    gate = torch.randn(3, h, d, dtype=torch.float64, requires_grad=True)
    acc, l, m = bt.attn_fwd_partial(q, k, v, blk, gate, None, score="gated", norm=norm)
    # autograd through an edge-list re-statement of the partials with m held constant
    src, dst = ei[0], ei[1]
    s = (q[dst] * k[src] * gate[et]).sum(-1) / d ** 0.5
    p = torch.exp(s - m.detach()[dst]) if norm == "softmax" else torch.exp(s.clamp(-5, 5))
    acc_r = torch.zeros_like(acc).index_add(0, dst, p.unsqueeze(-1) * v[src])
    l_r = torch.zeros_like(l).index_add(0, dst, p)
    assert (acc - acc_r).abs().max() < 1e-12 and (l - l_r).abs().max() < 1e-12
    dacc, dl = torch.randn_like(acc), torch.randn_like(l)
    ref = torch.autograd.grad((acc_r * dacc).sum() + (l_r * dl).sum(), [q, k, v, gate])
    got = bt.attn_bwd_partial(q.detach(), k.detach(), v.detach(), blk, gate.detach(), None, m, dacc, dl, score="gated", norm=norm)
    for a, b in zip(got[:4], ref):
        assert (a - b).abs().max() < 1e-11


def test_segments_and_csc_cover_all_edges():
    ei, et = random_graph(300, 5, seed=9)
    blk = BlockCSR.from_edges(ei, 300, 300, et)
    plan = blk.row_plan(16)
    assert int((plan.seg_end - plan.seg_beg).sum()) == blk.num_edges
    assert int((plan.seg_end - plan.seg_beg).max()) <= 16
    assert plan.num_slots == int((plan.seg_slot >= 0).sum())
    for i, r in enumerate(plan.split_rows.tolist()):
        a, b = plan.split_ptr[i].item(), plan.split_ptr[i + 1].item()
        segs = torch.nonzero((plan.seg_slot >= a) & (plan.seg_slot < b)).squeeze(1)
        assert (plan.seg_row[segs] == r).all()
    ccol, rowidx, et_t, pos, _ = blk.csc()
    assert (blk.col[pos.long()].long() == torch.repeat_interleave(torch.arange(300), (ccol[1:] - ccol[:-1]).long())).all()
    assert (blk.rows()[pos.long()] == rowidx).all() and (blk.etype[pos.long()] == et_t).all()
    cplan = blk.col_plan(16)
    assert int((cplan.seg_end - cplan.seg_beg).sum()) == blk.num_edges


@pytest.mark.parametrize("backend,parts", [("ref", (True, True)), ("torch", (True, True)), ("torch", (True, False)), ("torch", (False, True))])
def test_single_device_exphormer_matches_the_reference_model(backend, parts):
    """``Exphormer`` (stacked projection GEMM, CSR structures) against ``ExphormerRef`` (edge lists) with the same weights."""
    import torch
    from gt_b200.data.expander import random_regular_expander_edges
    from gt_b200.data.synthetic import add_self_loops, erdos_renyi, symmetrize
    from gt_b200.models.exphormer import AttentionGraph, Exphormer
    from gt_b200.models.exphormer_ref import ExphormerRef
    n, f, hid, classes = 50, 7, 16, 4
    with_attn, with_gcn = parts
    torch.manual_seed(1)
    ei = add_self_loops(symmetrize(erdos_renyi(n, 3, seed=5), n), n)
    exp = random_regular_expander_edges(n, 2, seed=2)
    x = torch.randn(n, f, dtype=torch.float64)
    kw = dict(dropout=0.0, gnn_dropout=0.0, with_gcn=with_gcn, with_attn=with_attn, norm="ln")
    ref = ExphormerRef(f, hid, classes, 2, 4, **kw).double()
    model = Exphormer(f, hid, classes, 2, 4, backend=backend, **kw).double()
    model.load_state_dict(ref.state_dict())
    graph = AttentionGraph(ei, exp, n, dtype=torch.float64)
    w = torch.randn(n, classes, dtype=torch.float64)
    out_ref, out = ref(x, ei, exp), model(x, graph)
    assert (out - out_ref).abs().max() < 1e-9
    (out_ref * w).sum().backward()
    (out * w).sum().backward()
    for (name, p), q in zip(model.named_parameters(), ref.parameters()):
        if q.grad is not None:
            assert (p.grad - q.grad).abs().max() < 1e-8, name
