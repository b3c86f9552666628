"""Density dispatch of the attention mask: the dense-tile / residual split (CPU) and the tensor-core tile kernel (GPU)."""
import pytest
import torch

from gt_b200.attention import BlockCSR
from gt_b200.attention import backend_torch as bt
from gt_b200.attention import tiles as tl


def clustered_block(n_rows, n_cols, cluster=128, p_in=0.3, n_sparse=2000, n_types=3, seed=0, clusters=None):
    """Communities of ``cluster`` nodes with dense internal masks plus a sparse random background; no duplicate edges."""
    g = torch.Generator().manual_seed(seed)
    dst, src = [], []
    n_cl = min(n_rows, n_cols) // cluster + 1
    for c in (range(n_cl) if clusters is None else clusters):
        r0, c0 = c * cluster, c * cluster
        rr, cc = min(n_rows, r0 + cluster) - r0, min(n_cols, c0 + cluster) - c0
        if rr <= 0 or cc <= 0:
            continue
        on = torch.rand(rr, cc, generator=g) < p_in
        d, s = on.nonzero(as_tuple=True)
        dst.append(d + r0); src.append(s + c0)
    dst.append(torch.randint(0, n_rows, (n_sparse,), generator=g)); src.append(torch.randint(0, n_cols, (n_sparse,), generator=g))
    dst, src = torch.cat(dst), torch.cat(src)
    key = torch.unique(dst * n_cols + src)
    dst, src = key // n_cols, key % n_cols
    et = torch.randint(0, n_types, (key.numel(),), generator=g)
    return BlockCSR.from_edges(torch.stack([src, dst]), n_rows, n_cols, et)


def merge(a, b, norm):
    (acc1, l1, m1), (acc2, l2, m2) = a, b
    if norm != "softmax":
        return acc1 + acc2, l1 + l2, m1
    m1e = torch.where(l1 > 0, m1, torch.full_like(m1, float("-inf")))
    m2e = torch.where(l2 > 0, m2, torch.full_like(m2, float("-inf")))
    m = torch.maximum(m1e, m2e)
    ms = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w1 = torch.where(l1 > 0, torch.exp(m1e - ms), torch.zeros_like(m))
    w2 = torch.where(l2 > 0, torch.exp(m2e - ms), torch.zeros_like(m))
    return acc1 * w1[..., None] + acc2 * w2[..., None], l1 * w1 + l2 * w2, ms


@pytest.mark.parametrize("score,norm", [("dot", "clampexp"), ("biased", "softmax"), ("dot", "softmax")])
def test_tile_split_is_exact(score, norm):
    torch.manual_seed(0)
    n, nc, h, d = 700, 600, 4, 32
    blk = clustered_block(n, nc)
    plan = tl.build_tile_plan(blk, min_edges=400, min_share=0.0)
    assert plan is not None and plan.num_tiles >= 4
    assert plan.num_tiled_edges + plan.residual.num_edges == blk.num_edges
    assert int((plan.mask != tl.NO_EDGE).sum()) == plan.num_tiled_edges
    assert plan.rb_ptr[-1] == plan.num_tiles and (plan.rb_ids[1:] > plan.rb_ids[:-1]).all()
    q, k, v = torch.randn(n, h, d), torch.randn(nc, h, d), torch.randn(nc, h, d)
    bias = torch.randn(3, h) if score == "biased" else None
    kw = dict(score=score, norm=norm)
    full = bt.attn_fwd_partial(q, k, v, blk, None, bias, **kw)
    part = merge(bt.attn_fwd_partial(q, k, v, plan.residual, None, bias, **kw), tl.tile_fwd_ref(q, k, v, plan, bias, **kw), norm)
    o_full, o_part = bt.normalize(full[0], full[1], norm), bt.normalize(part[0], part[1], norm)
    assert (o_full - o_part).abs().max() < 1e-4
    if norm == "clampexp":
        assert (full[1] - part[1]).abs().max() < 1e-3 * full[1].abs().max()


def test_tile_split_declines():
    blk = clustered_block(300, 300, p_in=0.01, n_sparse=500)
    assert tl.build_tile_plan(blk, min_edges=400, min_share=0.0) is None                 # no tile is dense enough
    dense = clustered_block(700, 600, clusters=[0], n_sparse=8000)
    assert tl.build_tile_plan(dense, min_edges=2000, min_share=0.5) is None              # dense tiles cover too little
    src = torch.tensor([0, 0, 1]); dst = torch.tensor([0, 0, 1])                         # a repeated edge cannot live in a byte map
    dup = BlockCSR.from_edges(torch.stack([src, dst]), 4, 4, torch.zeros(3, dtype=torch.long))
    assert tl.build_tile_plan(dup, min_edges=1, min_share=0.0) is None


# ---- GPU -----------------------------------------------------------------------------------------------------------------
def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / max(b.float().abs().max().item(), 1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("n,nc,h,score,norm", [
    (700, 600, 4, "dot", "clampexp"), (700, 600, 8, "biased", "softmax"), (1024, 1024, 16, "dot", "softmax"),
    (300, 900, 2, "biased", "clampexp"),
])
def test_tile_kernel_matches_oracle(n, nc, h, score, norm):
    from gt_b200.attention import backend_cuda as bc
    from gt_b200.ops import native
    dev = torch.device("cuda:0")
    torch.manual_seed(1)
    d = 32
    blk = clustered_block(n, nc, seed=2).to(dev)
    plan = tl.build_tile_plan(blk, min_edges=400, min_share=0.0)
    assert plan is not None
    q, k, v = (torch.randn(r, h, d, device=dev).bfloat16() for r in (n, nc, nc))
    bias = torch.randn(3, h, device=dev) if score == "biased" else None
    kw = dict(score=score, norm=norm)
    # 1. raw scores of the first tile (Q K^T on the tensor cores, before mask and scale)
    acc = torch.zeros(n, h, d, device=dev); l = torch.zeros(n, h, device=dev); m = torch.zeros(n, h, device=dev)
    dbg = torch.zeros(2, 128, 128, device=dev)
    bc.attn_tile_accumulate(q, k, v, plan, bias, acc, l, m, debug_scores=dbg, **kw)
    native.check_status(dev)
    r0, c0 = int(plan.rb_ids[0]) * 128, int(plan.tile_cb[0]) * 128
    r1, c1 = min(n, r0 + 128), min(nc, c0 + 128)
    s_ref = torch.einsum("rhd,chd->hrc", q[r0:r1, :2].float(), k[c0:c1, :2].float())
    assert _rel(dbg[:, :r1 - r0, :c1 - c0], s_ref) < 1e-3, "Q K^T"
    # 2. the tiles' partial states against the tile-by-tile oracle (zero initial state)
    acc_r, l_r, m_r = tl.tile_fwd_ref(q, k, v, plan, bias, **kw)
    if norm == "softmax":
        # (acc, l) are relative to the offset m, which may be any upper bound of the row maximum (the biased kernel uses
        # max(q.k) + max(bias)): compare the offset-free quantities
        on = l_r > 0
        assert ((l > 0) == on).all()
        assert ((l.log() + m)[on] - (l_r.log() + m_r)[on]).abs().max() < 2e-2, "log row sums"
        assert (m >= m_r - 1e-3).all()
        assert _rel(acc / l.clamp_min(1e-30)[..., None], acc_r / l_r.clamp_min(1e-30)[..., None]) < 2e-2, "P V"
    else:
        assert _rel(l, l_r) < 2e-2, "row sums"
        assert _rel(acc, acc_r) < 2e-2, "P V"
    # 3. merged into the gather kernels' state of the residual: equals the whole block on the gather kernels / the oracle
    full = bt.attn_fwd_partial(q.float(), k.float(), v.float(), blk, None, bias, **kw)
    blk._cache["tile_plan"] = plan
    got = bc.attn_fwd_partial(q, k, v, blk, None, bias, **kw)
    native.check_status(dev)
    o_ref, o_got = bt.normalize(full[0], full[1], norm), bt.normalize(got[0], got[1], norm)
    assert _rel(o_got, o_ref) < 2e-2
    assert _rel(got[1] * torch.exp(got[2]), full[1] * torch.exp(full[2])) < 2e-2 or norm == "softmax"
    # 4. the normalised operator with gradients: forward on both families, backward on the gather kernels
    qa, ka, va = (x.clone().float().requires_grad_() for x in (q, k, v))
    o_r = bt.masked_sparse_attention_torch(qa, ka, va, blk, bias=bias, **kw)
    w = torch.randn_like(o_r)
    gr = torch.autograd.grad((o_r * w).sum(), [qa, ka, va])
    qb, kb, vb = (x.clone().requires_grad_() for x in (q, k, v))
    o = bc.masked_sparse_attention_cuda(qb, kb, vb, blk, bias=bias, **kw)
    gg = torch.autograd.grad((o.float() * w).sum(), [qb, kb, vb])
    assert _rel(o, o_r) < 2e-2
    for a, b in zip(gg, gr):
        assert _rel(a, b) < 4e-2


def test_tile_split_without_edge_types_and_with_ragged_blocks():
    """Blocks without edge types (plain dot-product models) and with row / column counts that are not multiples of the tile."""
    torch.manual_seed(3)
    n, nc, h, d = 333, 517, 2, 32
    typed = clustered_block(n, nc, seed=5)
    blk = BlockCSR.from_csr(typed.crow, typed.col, None, n_cols=nc)
    plan = tl.build_tile_plan(blk, min_edges=300, min_share=0.0)
    assert plan is not None and plan.residual.etype is None
    assert int((plan.mask == 0).sum()) == plan.num_tiled_edges and int((plan.mask != tl.NO_EDGE).sum()) == plan.num_tiled_edges
    assert int(plan.tile_cb.max()) * 128 < nc and int(plan.rb_ids.max()) * 128 < n
    q, k, v = torch.randn(n, h, d), torch.randn(nc, h, d), torch.randn(nc, h, d)
    for norm in ("softmax", "clampexp"):
        full = bt.attn_fwd_partial(q, k, v, blk, None, None, score="dot", norm=norm)
        part = merge(bt.attn_fwd_partial(q, k, v, plan.residual, None, None, score="dot", norm=norm),
                     tl.tile_fwd_ref(q, k, v, plan, None, score="dot", norm=norm), norm)
        assert (bt.normalize(full[0], full[1], norm) - bt.normalize(part[0], part[1], norm)).abs().max() < 1e-4
    many = BlockCSR.from_csr(typed.crow, typed.col, typed.etype + 20, n_cols=nc)             # more edge types than a byte map encodes
    assert tl.build_tile_plan(many, min_edges=300, min_share=0.0) is None
