"""sm_100a kernels vs plain PyTorch fp32 references of the same op (run on a B200: ``pytest -m gpu``)."""
import itertools

import pytest
import torch

from helpers import random_graph

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda:0")


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / max(b.float().abs().max().item(), 1e-6)


@pytest.mark.parametrize("h,d,dtype,score,norm,seg", [
    (8, 32, torch.float32, "gated", "clampexp", 256), (8, 32, torch.bfloat16, "gated", "clampexp", 16),
    (4, 32, torch.float32, "dot", "softmax", 16), (16, 32, torch.float32, "biased", "softmax", 64),
    (4, 16, torch.float32, "gated", "softmax", 256), (2, 64, torch.bfloat16, "dot", "clampexp", 32),
    (1, 32, torch.float32, "biased", "clampexp", 256), (2, 40, torch.float32, "gated", "clampexp", 256),
])
def test_attention_fwd_bwd(h, d, dtype, score, norm, seg):
    from gt_b200.attention import BlockCSR
    from gt_b200.attention import backend_cuda as bc, backend_torch as bt
    dev = _dev()
    torch.manual_seed(0)
    n, t = 700, 3
    ei, et = random_graph(n, 6, seed=1)
    blk = BlockCSR.from_edges(ei, n, n, et).to(dev)
    q, k, v = (torch.randn(n, h, d, device=dev).to(dtype) for _ in range(3))
    gate, bias = torch.randn(t, h, d, device=dev), torch.randn(t, h, device=dev)
    kw = dict(score=score, norm=norm)
    g_, b_ = (gate if score == "gated" else None), (bias if score == "biased" else None)
    acc, l, m = bc.attn_fwd_partial(q, k, v, blk, g_, b_, seg_edges=seg, **kw)
    acc_r, l_r, m_r = bt.attn_fwd_partial(q.float(), k.float(), v.float(), blk, g_, b_, **kw)
    tol = 2e-4 if dtype == torch.float32 else 2e-2
    assert _rel(acc, acc_r) < tol and _rel(l, l_r) < tol and (m - m_r).abs().max() < tol * 10
    assert acc[3].abs().max() == 0 and l[7].abs().max() == 0
    dacc, dl = torch.randn_like(acc_r), torch.randn_like(l_r)
    got = bc.attn_bwd_partial(q, k, v, blk, g_, b_, m_r, dacc, dl, seg_edges=seg, **kw)
    ref = bt.attn_bwd_partial(q.float(), k.float(), v.float(), blk, g_, b_, m_r, dacc.to(dtype).float(), dl, **kw)
    for a, b, name in zip(got, ref, ("dq", "dk", "dv", "dgate", "dbias")):
        if b is not None:
            assert _rel(a, b) < (5e-4 if dtype == torch.float32 else 3e-2), name
    # normalised form through autograd
    qa, ka, va = (x.clone().float().requires_grad_() for x in (q, k, v))
    o_r = bt.masked_sparse_attention_torch(qa, ka, va, blk, gate=g_, bias=b_, **kw)
    w = torch.randn_like(o_r)
    gr = torch.autograd.grad((o_r * w).sum(), [qa, ka, va])
    qb, kb, vb = (x.clone().requires_grad_() for x in (q, k, v))
    o = bc.masked_sparse_attention_cuda(qb, kb, vb, blk, gate=g_, bias=b_, **kw)
    gg = torch.autograd.grad((o.float() * w).sum(), [qb, kb, vb])
    assert _rel(o, o_r) < tol
    for a, b in zip(gg, gr):
        assert _rel(a, b) < (5e-4 if dtype == torch.float32 else 4e-2)


def test_attention_accumulate_into_strided_payload():
    from gt_b200.attention import BlockCSR
    from gt_b200.attention import backend_cuda as bc, backend_torch as bt
    dev = _dev()
    torch.manual_seed(1)
    n, nc, h, d = 500, 300, 4, 32
    g = torch.Generator().manual_seed(3)
    src, dst = torch.randint(0, nc, (400,), generator=g), torch.randint(0, n, (400,), generator=g)   # most rows empty
    src = torch.cat([src, torch.arange(nc)]); dst = torch.cat([dst, torch.full((nc,), 5)])            # plus a hub row
    et = torch.randint(0, 2, (src.numel(),), generator=g)
    blk = BlockCSR.from_edges(torch.stack([src, dst]), n, nc, et).to(dev)
    q = torch.randn(n, h, d, device=dev).bfloat16()
    k, v = torch.randn(nc, h, d, device=dev).bfloat16(), torch.randn(nc, h, d, device=dev).bfloat16()
    gate = torch.randn(2, h, d, device=dev)
    hd = h * d
    packed = torch.randn(n, hd + h + 24, device=dev)
    before = packed.clone()
    bc.attn_fwd_partial_accum(q, k, v, blk, gate, None, packed, hd, seg_edges=64)
    acc_r, l_r, _ = bt.attn_fwd_partial(q.float(), k.float(), v.float(), blk, gate, None, score="gated", norm="clampexp")
    assert _rel(packed[:, :hd] - before[:, :hd], acc_r.reshape(n, hd)) < 2e-2
    assert _rel(packed[:, hd:hd + h] - before[:, hd:hd + h], l_r) < 2e-2
    assert torch.equal(packed[:, hd + h:], before[:, hd + h:])


def test_attention_backward_accumulates_dq_in_place():
    """Compact-accumulate backward: dq of the rows that own an edge is added into an fp32 buffer (hub row cut into segments,
    most rows empty and therefore untouched); dk / dv / dgate equal those of the plain partial backward."""
    from gt_b200.attention import BlockCSR
    from gt_b200.attention import backend_cuda as bc
    dev = _dev()
    torch.manual_seed(2)
    n, nc, h, d = 500, 300, 8, 32
    g = torch.Generator().manual_seed(5)
    src, dst = torch.randint(0, nc, (400,), generator=g), torch.randint(0, n, (400,), generator=g)
    src = torch.cat([src, torch.arange(nc)]); dst = torch.cat([dst, torch.full((nc,), 7)])
    et = torch.randint(0, 3, (src.numel(),), generator=g)
    blk = BlockCSR.from_edges(torch.stack([src, dst]), n, nc, et).to(dev)
    q = torch.randn(n, h, d, device=dev).bfloat16()
    k, v = torch.randn(nc, h, d, device=dev).bfloat16(), torch.randn(nc, h, d, device=dev).bfloat16()
    gate = torch.randn(3, h, d, device=dev)
    dacc, dl = torch.randn(n, h, d, device=dev), torch.randn(n, h, device=dev)
    m0 = torch.zeros(n, h, device=dev)
    kw = dict(score="gated", norm="clampexp", seg_edges=64)
    dq_r, dk_r, dv_r, dg_r, _ = bc.attn_bwd_partial(q, k, v, blk, gate, None, m0, dacc, dl, **kw)
    base = torch.randn(n, h * d, device=dev)
    buf = base.clone()
    dk, dv, dg, _ = bc.attn_bwd_partial_accum(q, k, v, blk, gate, None, m0, dacc, dl, buf, **kw)
    assert _rel(buf - base, dq_r.float().reshape(n, h * d)) < 2e-2
    empty = (blk.crow[1:] - blk.crow[:-1]) == 0
    assert torch.equal(buf[empty], base[empty])                     # rows without an edge are not touched
    assert _rel(dk, dk_r) < 1e-3 and _rel(dv, dv_r) < 1e-3 and _rel(dg, dg_r) < 1e-3


@pytest.mark.parametrize("d,dtype", [(256, torch.bfloat16), (128, torch.float32), (80, torch.float32), (512, torch.bfloat16)])
def test_spmm(d, dtype):
    from gt_b200.attention import BlockCSR
    from gt_b200.ops.sparse import spmm_raw
    dev = _dev()
    ei, _ = random_graph(900, 5, seed=2)
    w = torch.rand(ei.shape[1])
    blk = BlockCSR.from_edges(ei, 900, 900, weight=w)
    x = torch.randn(900, d)
    ref, ref_t = spmm_raw(blk, x), spmm_raw(blk, x, transpose=True)
    bg = blk.to(dev)
    xg = x.to(dev).to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert _rel(spmm_raw(bg, xg).cpu(), ref) < tol
    assert _rel(spmm_raw(bg, xg, transpose=True).cpu(), ref_t) < tol


@pytest.mark.parametrize("m,n,k", [(300, 256, 256), (1000, 512, 256), (129, 40, 128), (4096, 1024, 512), (77, 256, 64), (260, 136, 96)])
def test_gemm_nt_matches_fp32(m, n, k):
    from gt_b200.ops import native
    dev = _dev()
    torch.manual_seed(0)
    a, b = torch.randn(m, k, device=dev).bfloat16(), torch.randn(n, k, device=dev).bfloat16()
    bias = torch.randn(n, device=dev)
    ref = a.float() @ b.float().t()
    out = native.gemm_nt(a, b)
    torch.cuda.synchronize(); native.check_status(dev)
    assert _rel(out, ref) < 1e-2
    out32 = native.gemm_nt(a, b, bias, "relu", out_dtype=torch.float32)
    assert _rel(out32, torch.relu(ref + bias)) < 2e-3
    acc = torch.ones(m, n, device=dev)
    native.gemm_nt(a, b, out=acc, accumulate=True)
    assert _rel(acc, ref + 1) < 2e-3
    native.check_status(dev)


@pytest.mark.parametrize("m,n,k", [(1000, 256, 256), (5000, 512, 128), (64, 128, 256), (3001, 1024, 256), (333, 40, 136)])
def test_gemm_tn_matches_fp32(m, n, k):
    from gt_b200.ops import native
    dev = _dev()
    torch.manual_seed(0)
    a, b = torch.randn(m, n, device=dev).bfloat16(), torch.randn(m, k, device=dev).bfloat16()
    ref = a.float().t() @ b.float()
    out = native.gemm_tn(a, b)
    torch.cuda.synchronize(); native.check_status(dev)
    assert _rel(out, ref) < 2e-3
    native.gemm_tn(a, b, out=out, accumulate=True)
    assert _rel(out, 2 * ref) < 2e-3


def test_linear_autograd_and_dropout():
    from gt_b200.ops import functional as K, native
    dev = _dev()
    torch.manual_seed(0)
    x = torch.randn(600, 256, device=dev).bfloat16().requires_grad_()
    w = (torch.randn(512, 256, device=dev) * 0.05).requires_grad_()
    b = torch.randn(512, device=dev).requires_grad_()
    y = K.linear(x, w, b, activation="relu")
    xr, wr, br = x.detach().float().requires_grad_(), w.detach().bfloat16().float().requires_grad_(), b.detach().clone().requires_grad_()
    yr = torch.relu(xr @ wr.t() + br)
    g = torch.randn_like(yr)
    y.backward(g.bfloat16()); yr.backward(g.bfloat16().float())
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xr.grad) < 2e-2 and _rel(w.grad, wr.grad) < 2e-2 and _rel(b.grad, br.grad) < 2e-2
    native.seed_rng(7, dev)
    yd = K.linear(x.detach(), w.detach(), b.detach(), activation="relu", dropout=0.25, training=True)
    yd2 = K.linear(x.detach(), w.detach(), b.detach(), activation="relu", dropout=0.25, training=True)
    assert torch.equal(yd, yd2)                                   # same step, same site -> same mask
    kept = (yd != 0).float().sum() / (y != 0).float().sum()
    assert 0.72 < kept.item() < 0.78
    nz = yd != 0
    assert _rel(yd[nz], (y.detach().float() / 0.75)[nz]) < 1e-2


@pytest.mark.parametrize("d,dtype,p", [(256, torch.bfloat16, 0.0), (128, torch.float32, 0.0), (512, torch.float32, 0.2), (80, torch.float32, 0.0)])
def test_layer_norm_fused(d, dtype, p):
    from gt_b200.ops import native
    dev = _dev()
    torch.manual_seed(0)
    n = 333
    y, x = torch.randn(n, d, device=dev).to(dtype).requires_grad_(), torch.randn(n, d, device=dev).to(dtype).requires_grad_()
    yb, gam, bet = (torch.randn(d, device=dev).requires_grad_() for _ in range(3))
    native.seed_rng(3, dev)
    out = native.layer_norm(y, x, yb, gam, bet, 1e-5, p)
    g = torch.randn(n, d, device=dev)
    out.backward(g.to(dtype))
    if p == 0:
        y2, x2, yb2, gam2, bet2 = (t.detach().float().requires_grad_() for t in (y, x, yb, gam, bet))
        ref = torch.nn.functional.layer_norm(x2 + y2 + yb2, (d,), gam2, bet2, 1e-5)
        ref.backward(g.to(dtype).float())
        tol = 1e-4 if dtype == torch.float32 else 3e-2
        assert _rel(out, ref) < tol
        for a, b in ((y.grad, y2.grad), (x.grad, x2.grad), (yb.grad, yb2.grad), (gam.grad, gam2.grad), (bet.grad, bet2.grad)):
            assert _rel(a, b) < tol * 3
    else:
        # dropout: dy must be zero exactly where the mask dropped, and dx is the undropped LayerNorm gradient
        frac = (y.grad == 0).float().mean().item()
        assert abs(frac - p) < 0.03
        assert torch.isfinite(out).all() and (x.grad != 0).float().mean() > 0.99


def test_cross_entropy_and_adamw():
    from gt_b200.ops import native
    from gt_b200.ops.loss import masked_cross_entropy
    dev = _dev()
    torch.manual_seed(0)
    n, c = 500, 40
    lg = torch.randn(n, c, device=dev, requires_grad=True)
    y = torch.randint(0, c, (n,), device=dev)
    mask = torch.rand(n, device=dev) < 0.5
    loss = masked_cross_entropy(lg, y, mask, 123.0)
    loss.backward()
    lr_ = lg.detach().clone().requires_grad_()
    ref = torch.nn.functional.cross_entropy(lr_[mask], y[mask], reduction="sum") / 123.0
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-4 * abs(ref.item()) and _rel(lg.grad, lr_.grad) < 1e-5
    # AdamW with clipping vs torch.optim.AdamW + clip_grad_norm_
    p = torch.randn(1000, device=dev)
    pr = p.clone().requires_grad_()
    opt = torch.optim.AdamW([pr], lr=1e-2, weight_decay=0.1)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    hyper = torch.zeros(9, device=dev)
    e = native.ext()
    for t in range(1, 4):
        g = torch.randn(1000, device=dev) * 3
        pr.grad = g.clone()
        torch.nn.utils.clip_grad_norm_([pr], 1.0)
        opt.step()
        hyper[:8] = torch.tensor([1e-2, 0.9, 0.999, 1e-8, 0.1, 1 - 0.9 ** t, 1 - 0.999 ** t, 1.0], device=dev)
        hyper[8:9].zero_()
        e.sq_norm(g, hyper[8:9])
        e.adamw_step(p, g, m, v, None, hyper, None)
    assert _rel(p, pr.detach()) < 1e-5


def test_smoke_step_runs():
    """The smoke entry point (two bf16 steps of a tiny Exphormer) finishes with a finite loss and a clean status word; the
    comparison with the CPU oracle and the graph-replay check live in test_gpu_parity.py."""
    from gt_b200.train.engine import smoke_step
    smoke_step(_dev())


def test_layer_norm_with_fused_attention_normalisation():
    from gt_b200.ops import native
    dev = _dev()
    torch.manual_seed(0)
    n, h, dh = 257, 8, 32
    d = h * dh
    acc = torch.randn(n, d, device=dev, requires_grad=True)
    l = (torch.rand(n, h, device=dev) * 3).requires_grad_()
    x = torch.randn(n, d, device=dev).bfloat16().requires_grad_()
    gam, bet = torch.randn(d, device=dev).requires_grad_(), torch.randn(d, device=dev).requires_grad_()
    out = native.layer_norm(acc, x, None, gam, bet, 1e-5, 0.0, l, 1e-6)
    g = torch.randn(n, d, device=dev)
    out.backward(g.bfloat16())
    a2, l2, x2, g2, b2 = (t.detach().float().requires_grad_() for t in (acc, l, x, gam, bet))
    o = (a2.view(n, h, dh) / (l2 + 1e-6).unsqueeze(-1)).reshape(n, d)
    ref = torch.nn.functional.layer_norm(x2 + o, (d,), g2, b2, 1e-5)
    ref.backward(g.bfloat16().float())
    assert _rel(out, ref) < 2e-2
    for a, b, name in ((acc.grad, a2.grad, "dacc"), (l.grad, l2.grad, "dl"), (x.grad, x2.grad, "dx"), (gam.grad, g2.grad, "dgamma")):
        assert _rel(a, b) < 3e-2, name


def test_pack_and_unpack_columns():
    from gt_b200.ops import native
    DEV = _dev()
    torch.manual_seed(0)
    a = torch.randn(1001, 256, device=DEV)
    l = torch.rand(1001, 8, device=DEV)
    e = torch.randn(1001, 264, device=DEV).bfloat16()[:, :256]              # a strided view: row stride 264
    for wire in (torch.bfloat16, torch.float32):
        packed = native.pack_columns([a, l, e], wire)
        ref = torch.cat([a, l, e.float()], dim=1).to(wire)
        assert torch.equal(packed, ref)
        a2, l2, e2 = native.unpack_columns(packed, [256, 8, 256], [torch.float32, torch.float32, torch.bfloat16])
        assert torch.equal(a2, ref[:, :256].float()) and torch.equal(l2, ref[:, 256:264].float()) and torch.equal(e2, ref[:, 264:].bfloat16())
    native.check_status(DEV)


def test_head_dim_40_runs_on_the_kernels_with_padded_heads():
    """2 heads x 40 (the GraphGPS Exphormer recipe): forward and backward against the edge-list oracle in fp64."""
    from gt_b200.attention import BlockCSR, masked_sparse_attention_ref
    from gt_b200.attention.backend_cuda import _padded_dim, masked_sparse_attention_cuda
    dev = _dev()
    torch.manual_seed(0)
    n, h, d, t = 300, 2, 40, 2
    ei = torch.randint(0, n, (2, 2500))
    et = torch.randint(0, t, (2500,))
    q, k, v = (torch.randn(n, h, d, device=dev, requires_grad=True) for _ in range(3))
    gate = torch.randn(t, h, d, device=dev, requires_grad=True)
    assert _padded_dim(q, gate, None) == 64
    blk = BlockCSR.from_edges(ei, n, n, et).to(dev)
    o = masked_sparse_attention_cuda(q, k, v, blk, gate=gate, score="gated", norm="clampexp")
    w = torch.randn_like(o)
    (o * w).sum().backward()
    leaves = [x.detach().double().cpu().requires_grad_() for x in (q, k, v, gate)]
    o_ref = masked_sparse_attention_ref(leaves[0], leaves[1], leaves[2], ei, edge_type=et, gate=leaves[3], score="gated", norm="clampexp")
    (o_ref * w.double().cpu()).sum().backward()
    assert _rel(o.cpu(), o_ref) < 2e-4
    for a_, b_ in zip((q, k, v, gate), leaves):
        assert _rel(a_.grad.cpu(), b_.grad) < 5e-4


@pytest.mark.parametrize("l2norm,d", [(True, 256), (False, 128), (True, 512)])
def test_fused_input_stage_matches_torch(l2norm, d):
    import torch.nn.functional as F
    from gt_b200.ops import native
    dev = _dev()
    torch.manual_seed(0)
    n = 777
    h = torch.randn(n, d, device=dev, requires_grad=True)
    gamma = (torch.rand(d, device=dev) + 0.5).requires_grad_()
    beta = (torch.randn(d, device=dev) * 0.1).requires_grad_()
    w = torch.randn(n, d, device=dev)
    out = native.pre_mp(h, gamma, beta, 1e-5, 0.0, l2norm)
    (out * w).sum().backward()
    got = [out.detach().clone(), h.grad.clone(), gamma.grad.clone(), beta.grad.clone()]
    h.grad = gamma.grad = beta.grad = None
    ref = F.relu(F.layer_norm(h, (d,), gamma, beta, 1e-5))
    ref = F.normalize(ref, p=2, dim=1) if l2norm else ref
    (ref * w).sum().backward()
    for a_, b_ in zip(got, (ref.detach(), h.grad, gamma.grad, beta.grad)):
        assert _rel(a_, b_) < 2e-4
    # dropout: the backward regenerates the forward's mask (gradient is zero exactly where the output is zero)
    hb = torch.randn(n, d, device=dev).bfloat16().requires_grad_()
    ob = native.pre_mp(hb, gamma, beta, 1e-5, 0.3, l2norm)
    ob.sum().backward()
    dropped = (ob == 0).float().mean().item()
    assert 0.55 < dropped < 0.75                                   # ~half by ReLU of what 30 % dropout leaves
    native.check_status(dev)


def test_embed_add_and_gated_residual_kernels():
    import torch.nn as nn
    from gt_b200.ops import functional as K
    dev = _dev()
    torch.manual_seed(0)
    n, d = 1003, 128
    # embedding lookups folded into one pass (padding index adds nothing), gradients of the tables by atomics
    x = torch.randn(n, d, device=dev, requires_grad=True)
    ea, eb = nn.Embedding(20, d, padding_idx=19).to(dev), nn.Embedding(7, d).to(dev)
    ia, ib = torch.randint(0, 20, (n,), device=dev), torch.randint(0, 7, (n,), device=dev)
    w = torch.randn(n, d, device=dev)
    out = K.embed_add(x, ea, ia, eb, ib)
    (out * w).sum().backward()
    got = [out.detach().clone(), x.grad.clone(), ea.weight.grad.clone(), eb.weight.grad.clone()]
    x.grad = None; ea.weight.grad = None; eb.weight.grad = None
    ref = x + ea(ia) + eb(ib)
    (ref * w).sum().backward()
    for a_, b_ in zip(got, (ref.detach(), x.grad, ea.weight.grad, eb.weight.grad)):
        assert _rel(a_, b_) < 1e-5
    # UniMP gated residual vs the composed torch expression
    r = torch.randn(n, d, device=dev, requires_grad=True)
    o = torch.randn(n, d, device=dev, requires_grad=True)
    gate, ln = nn.Linear(3 * d, 1).to(dev), K.LayerNorm(d).to(dev)
    with torch.no_grad():
        ln.weight.uniform_(0.5, 1.5); ln.bias.normal_(0, 0.1)
    out = K.gated_residual(r, o, gate.weight, gate.bias, ln, 0.0, True)
    (out * w).sum().backward()
    params = (r, o, gate.weight, gate.bias, ln.weight, ln.bias)
    got = [out.detach().clone()] + [p_.grad.clone() for p_ in params]
    for p_ in params:
        p_.grad = None
    beta = torch.sigmoid(gate(torch.cat([r, o, r - o], dim=1)))
    ref = torch.relu(torch.nn.functional.layer_norm(beta * r + (1 - beta) * o, (d,), ln.weight, ln.bias, ln.eps))
    (ref * w).sum().backward()
    for a_, b_ in zip(got, [ref.detach()] + [p_.grad for p_ in params]):
        assert _rel(a_, b_) < 5e-4
