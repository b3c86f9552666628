"""Peer-memory collectives and the distributed model on >= 2 real GPUs (NCCL for bootstrap and as the comparison).
Child processes, one per GPU; skipped when the box has a single GPU."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _spawn(fn, world, *args):
    import tempfile
    import torch.multiprocessing as mp
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(fn, args=(world, os.path.join(tmp, "store")) + args, nprocs=world, join=True)


def _init(rank, world, store):
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"file://{store}", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    return torch.device("cuda", rank)


def _collectives_worker(rank, world, store):
    import torch.distributed as dist
    from gt_b200.ops import native
    from gt_b200.parallel.sparse_comm import SparseRowPlan
    from gt_b200.parallel.symm import SymmetricHeap
    dev = _init(rank, world, store)
    heap = SymmetricHeap(dev, 256 << 20)
    torch.manual_seed(rank)
    for dtype in (torch.float32, torch.bfloat16):
        for rep in range(3):                       # repeated use of the same call sites (staging reuse across "steps")
            heap.begin_step()
            x = torch.randn(1000, 64, device=dev).to(dtype)
            ref = torch.empty(world * 1000, 64, device=dev, dtype=dtype)
            dist.all_gather_into_tensor(ref, x)
            assert torch.equal(heap.all_gather(x, None), ref)
            y = torch.randn(world * 504, 72, device=dev).to(dtype)
            ref = torch.empty(504, 72, device=dev, dtype=torch.float32)
            dist.reduce_scatter_tensor(ref, y.float())
            got = heap.reduce_scatter(y, None)
            assert (got.float() - ref).abs().max() < (1e-5 if dtype == torch.float32 else 0.1)
    g = heap.empty(4096, torch.float32, "grads")
    out = torch.empty_like(g)
    for rep in range(2):
        heap.begin_step()
        g.copy_(torch.randn(4096, device=dev))
        ref = g.clone()
        dist.all_reduce(ref)
        heap.all_reduce(g, out, "grads")
        assert (out - ref).abs().max() < 1e-5
    # several column blocks reduced in one packed payload (forward) / gathered (backward) vs the concatenated reference
    from gt_b200.parallel.attention import _PackedReduceScatter
    from gt_b200.parallel.collectives import reduce_scatter_rows
    heap.begin_step()
    acc = torch.randn(world * 512, 64, device=dev, requires_grad=True)
    l = torch.rand(world * 512, 8, device=dev, requires_grad=True)
    ex = torch.randn(world * 512, 32, device=dev).bfloat16().requires_grad_()
    o = _PackedReduceScatter.apply(None, torch.bfloat16, acc, l, ex)
    w = [torch.randn_like(t) for t in o]
    sum((a_ * b_).sum() for a_, b_ in zip(o, w)).backward()
    got = [acc.grad.clone(), l.grad.clone(), ex.grad.clone()]
    acc.grad = l.grad = ex.grad = None
    ref = reduce_scatter_rows(torch.cat([acc, l, ex.float()], dim=1), None, torch.bfloat16)
    assert (torch.cat([o[0], o[1], o[2].float()], dim=1) - ref).abs().max() < 0.1
    (ref * torch.cat([w[0], w[1], w[2].float()], dim=1)).sum().backward()
    for g_, r_ in zip(got, (acc.grad, l.grad, ex.grad)):
        assert (g_.float() - r_.float()).abs().max() < 0.05
    # Ulysses all-to-all by strided peer reads vs the NCCL all-to-all with transposes
    from gt_b200.parallel.collectives import raw_heads_to_rows, raw_rows_to_heads, set_transport
    xa = torch.randn(96, 4 * world, 16, device=dev).bfloat16()
    set_transport(None)
    ref_h = raw_rows_to_heads(xa, None, world)
    ref_r = raw_heads_to_rows(ref_h, None, world)
    set_transport(heap)
    heap.begin_step()
    got_h = raw_rows_to_heads(xa, None, world)
    got_r = raw_heads_to_rows(got_h, None, world)
    set_transport(None)
    assert torch.equal(got_h, ref_h) and torch.equal(got_r, ref_r) and torch.equal(got_r, xa)
    # statistics all-reduce (BatchNorm sums) by the one-shot peer kernel, forward and backward, vs NCCL
    from gt_b200.parallel.collectives import all_reduce_sum
    st = torch.randn(4 * 64, device=dev)
    res = {}
    for name, tr in (("nccl", None), ("p2p", heap)):
        set_transport(tr)
        heap.begin_step()
        leaf = st.clone().requires_grad_()
        y = all_reduce_sum(leaf)
        (y * (rank + 1.0)).sum().backward()
        res[name] = (y.detach().clone(), leaf.grad.clone())
    set_transport(None)
    assert (res["p2p"][0] - res["nccl"][0]).abs().max() < 1e-5 and (res["p2p"][1] - res["nccl"][1]).abs().max() < 1e-5
    assert abs(float(res["p2p"][1][0]) - world * (world + 1) / 2) < 1e-5
    # sparse plan: pull transport vs all-to-all-v transport
    need = torch.unique(torch.randint(0, world * 300, (200,), device=dev))
    plan_a = SparseRowPlan(None, 300, need, "t", "a2a")
    plan_p = SparseRowPlan(None, 300, need, "t", "pull", heap)
    for rep in range(2):
        heap.begin_step()
        x = torch.randn(300, 64, device=dev).bfloat16()
        assert torch.equal(plan_p.gather(x), plan_a.gather(x))
        yv = torch.randn(plan_a.n_need, 64, device=dev)
        assert (plan_p.reduce_scatter(yv) - plan_a.reduce_scatter(yv)).abs().max() < 1e-4
    torch.cuda.synchronize()
    native.check_status(dev)
    dist.barrier()
    dist.destroy_process_group()


def _fused_gemm_worker(rank, world, store):
    """All-gather fused into the GEMM (TMA loads from peer memory) and reduce-scatter fused into the GEMM epilogue (peer
    stores) against the unfused NCCL + GEMM pair, forward and backward, on shapes with ragged tile edges."""
    import torch.distributed as dist
    from gt_b200.ops import native
    from gt_b200.parallel.collectives import all_gather_rows, set_transport
    from gt_b200.parallel.fused_comm import fused_ok, linear_gather
    from gt_b200.parallel.symm import SymmetricHeap
    dev = _init(rank, world, store)
    heap = SymmetricHeap(dev, 512 << 20)
    for chunk, k, n in ((1000, 256, 768), (4104, 128, 256), (520, 512, 136), (37000, 256, 768)):
        torch.manual_seed(7)
        w = (torch.randn(n, k, device=dev) * k ** -0.5).requires_grad_()
        torch.manual_seed(100 + rank)
        x = torch.randn(chunk, k, device=dev).bfloat16().requires_grad_()
        gy = torch.randn(world * chunk, n, device=dev).bfloat16()
        set_transport(None)
        ref = native.linear(all_gather_rows(x, None), w)
        ref.backward(gy)
        gx_ref, gw_ref = x.grad.clone(), w.grad.clone()
        x.grad = w.grad = None
        set_transport(heap)
        assert fused_ok(x, w, None)
        for rep in range(2):                                    # twice: the staging buffers of a call site are reused
            heap.begin_step()
            out = linear_gather(x, w, None)
            out.backward(gy)
            assert (out.float() - ref.float()).abs().max() <= 2e-2 * ref.float().abs().max(), (chunk, k, n)
            assert (x.grad.float() - gx_ref.float()).abs().max() <= 3e-2 * gx_ref.float().abs().max() + 1e-3, (chunk, k, n)
            assert (w.grad - gw_ref).abs().max() <= 2e-2 * gw_ref.abs().max() + 1e-3, (chunk, k, n)
            x.grad = w.grad = None
        # the gathered by-product equals the all-gather
        heap.begin_step()
        y, xg = heap.linear_gather(x.detach(), w.detach().bfloat16(), None, want_gathered=True)
        set_transport(None)
        assert torch.equal(xg, all_gather_rows(x.detach(), None))
    torch.cuda.synchronize()
    native.check_status(dev)
    set_transport(None)
    dist.barrier()
    dist.destroy_process_group()


def _pull_attention_worker(rank, world, store):
    """Attention whose kernel pulls K / V rows from the owners' memory vs the gathered-operand operator (forward and backward)."""
    import torch.distributed as dist
    from gt_b200.ops import native
    from gt_b200.parallel import attention as pa
    from gt_b200.parallel.collectives import all_gather_rows, set_transport
    from gt_b200.parallel.grid import make_grid
    from gt_b200.parallel.symm import SymmetricHeap
    dev = _init(rank, world, store)
    heap = SymmetricHeap(dev, 256 << 20)
    set_transport(heap)
    n, h, d = 4096, 4, 32
    g = torch.Generator().manual_seed(3)
    ei = torch.randint(0, n, (2, 40000), generator=g)
    et = torch.randint(0, 2, (40000,), generator=g)
    grid = make_grid((world, 1), n, n_pad=n).to(dev)
    b_ei, b_et = grid.local_block(ei, et)
    block = pa.AttentionBlock(grid, b_ei.to(dev), b_et.to(dev))
    torch.manual_seed(rank)
    q, k, v = (torch.randn(grid.chunk, h, d, device=dev).bfloat16().requires_grad_() for _ in range(3))
    gate = torch.randn(2, h, d, device=dev, requires_grad=True)
    ref_op = pa.DistAttentionPartial(grid, block, h, d)
    pull_op = pa.DistAttentionPullKV(grid, block, h, d, heap)
    outs = {}
    for name in ("ref", "pull"):
        heap.begin_step()
        if name == "ref":
            acc, l, m = ref_op(q, all_gather_rows(k, grid.col_group), all_gather_rows(v, grid.col_group), gate)
        else:
            acc, l, m = pull_op(q, k, v, gate)
        ((acc * 0.01).sum() + l.sum()).backward()
        outs[name] = [t.detach().float().clone() for t in (acc, l, q.grad, k.grad, v.grad, gate.grad)]
        q.grad = k.grad = v.grad = gate.grad = None
    for a_, b_ in zip(outs["ref"], outs["pull"]):
        assert (a_ - b_).abs().max() <= 2e-2 * a_.abs().max() + 1e-4
    torch.cuda.synchronize()
    native.check_status(dev)
    set_transport(None)
    dist.barrier()
    dist.destroy_process_group()


def _model_worker(rank, world, store, grid_shape):
    import torch.distributed as dist
    from gt_b200.ops import native
    from gt_b200.parallel.collectives import set_transport
    from gt_b200.parallel.layers import dist_cross_entropy
    from gt_b200.parallel.symm import SymmetricHeap
    from gt_b200.train.engine import TrainEngine
    from gt_b200.train.workloads import exphormer_workload
    dev = _init(rank, world, store)
    losses = {}
    for comm in ("nccl", "p2p"):
        heap = SymmetricHeap(dev, 512 << 20) if comm == "p2p" else None
        set_transport(heap)
        wl = exphormer_workload("exphormer_arxiv", grid_shape, dev, torch.bfloat16, scale_down=32, layers=2, hidden=128, heads=4,
                                dropout=0.0, heap=heap)
        model = wl["model"]
        for p in model.parameters():
            dist.broadcast(p.data, src=0)
        eng = TrainEngine(model, total_steps=10, warmup=1, heap=heap, use_graph=(comm == "p2p"), graph_warmup=2)
        x, y, m = wl["x"].to(dev), wl["y"].to(dev), wl["masks"]["train"].to(dev)
        out = []
        for _ in range(5):
            out.append(eng.train_step(lambda: dist_cross_entropy(model(x), y, m, wl["n_train"])).clone())
        torch.cuda.synchronize()
        native.check_status(dev)
        tot = torch.stack(out)
        dist.all_reduce(tot)
        losses[comm] = tot.cpu()
        set_transport(None)
    assert torch.isfinite(losses["p2p"]).all()
    assert (losses["p2p"] - losses["nccl"]).abs().max() < 5e-2, (losses["p2p"], losses["nccl"])
    assert losses["nccl"][-1] < losses["nccl"][0]
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_peer_memory_collectives_match_nccl():
    _spawn(_collectives_worker, 2)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_collective_fused_gemms_match_unfused():
    _spawn(_fused_gemm_worker, 2)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_attention_pulling_kv_from_peer_memory():
    _spawn(_pull_attention_worker, 2)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_dist_model_p2p_matches_nccl_2gpu():
    _spawn(_model_worker, 2, (2, 1))


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs >= 4 GPUs")
def test_dist_model_p2p_matches_nccl_4gpu():
    _spawn(_model_worker, 4, (2, 2))
