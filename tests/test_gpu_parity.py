"""Whole-model parity on GPUs with the native kernels: every layer kind and model variant against the single-process fp64
reference on the CPU (owned logits, loss, EVERY parameter gradient after the all-reduce, BatchNorm running statistics), on
1, 2 and 4 ranks, over NCCL and over the peer-memory transport, in fp32 and in bf16.  The cases mirror those the reference
checks on NCCL ranks (``gt3d/tests/test_dist_model.py:23-51``, tolerances ``:51``; operator level
``gt3d/tests/test_dist_attention.py:94``).  Multi-rank cases run as child processes, one per GPU, several cases per launch.
"""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

# (forward, gradient) error bounds relative to the largest reference magnitude
TOL = {torch.float32: (5e-4, 5e-3), torch.bfloat16: (3e-2, 2e-1)}

EXPHORMER_CASES = {
    "plain": dict(),
    "plain_ln": dict(norm="ln"),
    "fused": dict(fused=True),
    "fused_ln": dict(fused=True, norm="ln"),
    "fused_nogcn": dict(fused=True, with_gcn=False, norm="ln"),
    "fused_gather_proj": dict(fused=True, gather_proj=True),
    "fused_sparse": dict(fused=True, sparse_comm=True, sparse_threshold=1.0),
    "fused_ckpt": dict(fused=True, checkpoint=True, norm="ln"),
    "pipelined": dict(fused=True, pipeline_sub=2),
    "streamed": dict(fused=True, stream_sub=2),
    "streamed_sync_nocompact": dict(fused=True, stream_sub=2, stream_overlap=False, stream_compact=False),
    "ring": dict(ring=True),
    "head": dict(with_gcn=False),
    "head_gcn": dict(),
}


def _rel(a, b, floor=1e-6):
    return (a.double().cpu() - b.double().cpu()).abs().max().item() / max(b.double().abs().max().item(), floor)


def _grad_floor(ref_grads):
    """Errors are measured against at least 1 % of the largest gradient magnitude of the model."""
    return 1e-2 * max(float(p.grad.abs().max()) for p in ref_grads.values() if p.grad is not None)


def _grad_err(got, ref, floor):
    """A gradient that vanishes analytically (a bias in front of a batch normalisation: |ref| < 1e-3 of the largest gradient) is
    pure cancellation noise in low precision; it is measured against the largest gradient magnitude instead."""
    if float(ref.abs().max()) < 0.1 * floor:
        return _rel(got, ref, 100.0 * floor)
    return _rel(got, ref, floor)


def _exphormer_case(dev, grid_shape, name, dtype, heap):
    """One case on the current process group; raises AssertionError with the offending tensor's name."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import torch.distributed as dist
    from helpers import random_graph
    from gt_b200.data.expander import random_regular_expander_edges
    from gt_b200.models.exphormer_dist import DistExphormer
    from gt_b200.models.exphormer_ref import ExphormerRef, gcn_edges_with_self_loops
    from gt_b200.ops import native
    from gt_b200.parallel.collectives import set_transport
    from gt_b200.parallel.grid import make_grid
    from gt_b200.parallel.layers import dist_cross_entropy, set_step
    from gt_b200.train.engine import TrainEngine
    cfg = dict(EXPHORMER_CASES[name])
    world = dist.get_world_size()
    n, f, hid, classes, heads = 1000, 16, 64, 8, 4
    torch.manual_seed(0)
    ei, _ = random_graph(n, 4, seed=3, hub=True, empty=())
    ei = ei[:, ei[0] != ei[1]]
    exp = random_regular_expander_edges(n, 3, seed=1)
    x = torch.randn(n, f, dtype=torch.float64)
    y = torch.randint(0, classes, (n,))
    mask = torch.rand(n) < 0.6
    norm = cfg.get("norm", "bn")
    with_gcn = cfg.get("with_gcn", True)
    ref = ExphormerRef(f, hid, classes, 2, heads, dropout=0.0, gnn_dropout=0.0, with_gcn=with_gcn, norm=norm).double()
    n_pad = -(-n // (16 * world)) * (16 * world)
    grid = make_grid(grid_shape, n, n_pad=n_pad).to(dev)
    gcn_blk, _ = grid.local_block(gcn_edges_with_self_loops(ei, n))
    attn_ei, attn_et = ExphormerRef.build_attention_edges(ei, exp)
    a_blk, a_et = grid.local_block(attn_ei, attn_et)
    set_transport(heap)
    bf16 = dtype == torch.bfloat16
    kw = dict(comm_dtype=torch.bfloat16 if bf16 else None, rs_dtype=torch.bfloat16 if (bf16 and world > 1) else None,
              kernel_dtype=torch.bfloat16 if bf16 else None, heap=heap)
    if cfg.get("sparse_comm") and heap is not None:
        kw["sparse_transport"] = "pull"
    model = DistExphormer(grid, gcn_blk.to(dev), a_blk.to(dev), a_et.to(dev), f, hid, classes, 2, heads, dropout=0.0, gnn_dropout=0.0,
                          backend="cuda", **kw, **cfg)
    model.load_ref_state_dict(ref.state_dict())
    model = model.to(dev)
    eng = TrainEngine(model, heap=heap)                       # flat buffers, bf16 shadow, stacked views of the fused layers
    set_step(0)
    ref.train(); model.train()
    out_ref = ref(x, ei, exp)
    loss_ref = torch.nn.functional.cross_entropy(out_ref[mask], y[mask], reduction="sum") / int(mask.sum())
    loss_ref.backward()
    if world > 1:                       # ranks build their models at different speeds: start the step together
        torch.cuda.synchronize()
        dist.barrier()
    if heap is not None:
        heap.begin_step()
    eng.flat_g.zero_()
    out = model(grid.take_owned(x).to(dev).to(dtype))
    lo, hi = grid.owned_range()
    nv = max(min(hi, n) - lo, 0)
    tol_f, tol_g = TOL[dtype]
    scale = out_ref.abs().max().item()
    err = (out[:nv].double().cpu() - out_ref[lo:lo + nv]).abs().max().item() / scale if nv else 0.0
    # judged after the backward pass: a rank that raised here would skip the collectives its peers still wait for
    logit_err = err
    m_loc = (grid.take_owned(mask.to(torch.uint8)).bool() & grid.valid_mask.cpu()).to(dev)
    loss = dist_cross_entropy(out, grid.take_owned(y).to(dev), m_loc, int(mask.sum()))
    loss.backward()
    tot = loss.detach().float().clone()
    if world > 1:
        dist.all_reduce(tot)
        dist.all_reduce(eng.flat_g)
    assert logit_err < tol_f, (name, "logits", logit_err)
    assert abs(tot.item() - loss_ref.item()) < tol_f * max(1.0, abs(loss_ref.item())) * 4, (name, "loss", tot.item(), loss_ref.item())
    torch.cuda.synchronize()
    native.check_status(dev)
    ref_grads = dict(ref.named_parameters())
    worst = ("", 0.0)
    floor = _grad_floor(ref_grads)
    for pname, p in model.named_parameters():
        gr = ref_grads[pname].grad
        if gr is None:
            continue
        e_ = _grad_err(p.grad, gr, floor)
        if e_ > worst[1]:
            worst = (pname, e_)
    assert worst[1] < tol_g, (name, "gradient", worst)
    if norm == "bn":
        sd, rsd = model.state_dict(), ref.state_dict()
        for k_ in sd:
            if "running" in k_:
                assert _rel(sd[k_], rsd[k_]) < tol_f * 4, (name, k_)
    set_transport(None)


def _variant_case(dev, grid_shape, cfg, dtype, heap):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import torch.distributed as dist
    from helpers import random_graph
    from gt_b200.data.synthetic import degrees, symmetrize
    from gt_b200.models import gt_variants as gv
    from gt_b200.ops import native
    from gt_b200.parallel.collectives import set_transport
    from gt_b200.parallel.grid import make_grid
    from gt_b200.parallel.layers import dist_cross_entropy
    from gt_b200.train.engine import TrainEngine
    world = dist.get_world_size()
    n, f, hid, classes, heads = 999, 16, 64, 6, 4
    torch.manual_seed(0)
    ei, _ = random_graph(n, 3, seed=4, hub=True, empty=())
    ei = symmetrize(ei[:, ei[0] != ei[1]], n)
    x = torch.randn(n + 1, f, dtype=torch.float64)
    y = torch.randint(0, classes, (n + 1,))
    mask = torch.rand(n + 1) < 0.6
    mask[n] = False
    n_pad = -(-(n + 1) // (8 * world)) * (8 * world)
    grid = make_grid(grid_shape, n, n_pad=n_pad).to(dev)
    set_transport(heap)
    if cfg["model"] == "unimp":
        a_ei, a_et = gv.typed_graph_edges(ei, n)
        ref = gv.UniMPRef(f, hid, classes, 2, heads, dropout=0.0).double()
        out_ref = ref(x[:n], a_ei, None)
        kw, fw = {}, {}
    else:
        if cfg.get("khop"):
            a_ei, a_et = gv.khop_typed_edges(ei, n, max_two_hop=16, seed=0)
            nt, tok, outdeg = 3, None, True
            nb = a_ei[:, a_et == 1]
        else:
            a_ei, a_et = gv.graphormer_edges(ei, n)
            nt, tok, outdeg = 4, n, False
            nb = a_ei[:, a_et == 0]
        n_ref = n if cfg.get("khop") else n + 1
        ind, outd = degrees(nb, n_ref)
        ref = gv.GraphormerNodeRef(f, hid, classes, 2, heads, dropout=0.0, max_degree=16, num_edge_types=nt, out_degree=outdeg).double()
        with torch.no_grad():
            ref.attn_bias.normal_()
        out_ref = ref(x[:n_ref], a_ei, a_et, ind, tok, outd if outdeg else None)
        kw = dict(max_degree=16, num_edge_types=nt, out_degree=outdeg, token_row=gv.token_owned_row(grid, n) if tok is not None else None)
        b_ei, b_et = grid.local_block(a_ei, a_et)
        d_in, d_out = gv.owned_degrees(grid, b_ei.to(dev), b_et.to(dev), dev, neighbour_type=1 if cfg.get("khop") else 0)
        fw = dict(degree_loc=d_in, out_degree_loc=d_out if outdeg else None)
    b_ei, b_et = grid.local_block(a_ei, a_et)
    bf16 = dtype == torch.bfloat16
    model = gv.DistGTVariant(grid, b_ei.to(dev), b_et.to(dev), f, hid, classes, 2, heads, model=cfg["model"], dropout=0.0, backend="cuda",
                             comm_dtype=torch.bfloat16 if bf16 else None, rs_dtype=torch.bfloat16 if (bf16 and world > 1) else None, **kw)
    model.load_ref_state_dict(ref.state_dict())
    model = model.to(dev)
    eng = TrainEngine(model, heap=heap)
    nm = int(mask.sum())
    rows = out_ref.shape[0]
    loss_ref = torch.nn.functional.cross_entropy(out_ref[mask[:rows]], y[:rows][mask[:rows]], reduction="sum") / nm
    loss_ref.backward()
    model.train()
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
    if heap is not None:
        heap.begin_step()
    eng.flat_g.zero_()
    out = model(grid.take_owned(x).to(dev).to(dtype), **fw)
    lo, hi = grid.owned_range()
    nv = max(min(hi, rows) - lo, 0)
    tol_f, tol_g = TOL[dtype]
    err = (out[:nv].double().cpu() - out_ref[lo:lo + nv]).abs().max().item() / out_ref.abs().max().item() if nv else 0.0
    m_loc = grid.take_owned(mask.to(torch.uint8)).bool().to(dev)
    dist_cross_entropy(out, grid.take_owned(y).to(dev), m_loc, nm).backward()
    if world > 1:
        dist.all_reduce(eng.flat_g)
    torch.cuda.synchronize()
    assert err < tol_f, (cfg, "logits", err)              # after the backward pass, so that no rank leaves its peers waiting
    native.check_status(dev)
    rg = dict(ref.named_parameters())
    worst = ("", 0.0)
    floor = _grad_floor(rg)
    for pname, p in model.named_parameters():
        gr = rg[pname].grad
        if gr is None:
            continue
        e_ = _grad_err(p.grad, gr, floor)
        if e_ > worst[1]:
            worst = (pname, e_)
    assert worst[1] < tol_g, (cfg, "gradient", worst)
    set_transport(None)


# ---- one GPU ------------------------------------------------------------------------------------------------------------
ONE_GPU = ["plain", "plain_ln", "fused", "fused_ln", "fused_nogcn", "fused_ckpt", "pipelined", "streamed", "streamed_sync_nocompact"]


def _single():
    from gt_b200.train.engine import init_single_process_group
    torch.cuda.set_device(0)
    init_single_process_group()
    return torch.device("cuda", 0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", ONE_GPU)
def test_exphormer_layer_kinds_one_gpu(name, dtype):
    _exphormer_case(_single(), (1, 1), name, dtype, None)


@pytest.mark.parametrize("cfg", [dict(model="unimp"), dict(model="graphormer"), dict(model="graphormer", khop=True)],
                         ids=["unimp", "graphormer_token", "graphormer_khop"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_variants_one_gpu(cfg, dtype):
    _variant_case(_single(), (1, 1), cfg, dtype, None)


def test_whole_step_matches_cpu_oracle_and_graph_replay():
    """(1) One fp32 and one bf16 step of the flagship configuration against the fp64 CPU reference: logits, loss and every
    parameter gradient (the ``fused_ln`` cases above).  (2) A CUDA-graph replayed step equals an eager step: two engines with the
    same weights, seeds and dropout-RNG offsets, one eager and one captured, must report the same losses step by step."""
    from gt_b200.ops import native
    from gt_b200.parallel.layers import dist_cross_entropy
    from gt_b200.train.engine import TrainEngine
    from gt_b200.train.workloads import exphormer_workload
    dev = _single()
    losses = {}
    for mode in ("eager", "graph"):
        native.seed_rng(1234, dev)
        wl = exphormer_workload("exphormer_arxiv", (1, 1), dev, torch.bfloat16, scale_down=16, layers=2, hidden=128, heads=4, dropout=0.1)
        model = wl["model"]
        eng = TrainEngine(model, total_steps=8, warmup=1, use_graph=(mode == "graph"), graph_warmup=2)
        x, y, m = wl["x"].to(dev), wl["y"].to(dev), wl["masks"]["train"].to(dev)
        model.train()
        out = [eng.train_step(lambda: dist_cross_entropy(model(x), y, m, wl["n_train"])).clone() for _ in range(6)]
        torch.cuda.synchronize()
        native.check_status(dev)
        losses[mode] = torch.stack(out).cpu()
    assert torch.isfinite(losses["graph"]).all()
    assert losses["eager"][-1] < losses["eager"][0]
    # steps 0-1 of the captured engine ran eagerly, step 2 is the capture, 3-5 are replays
    assert (losses["graph"] - losses["eager"]).abs().max() < 2e-3, (losses["graph"], losses["eager"])


def test_resume_with_cuda_graph_matches_uninterrupted(tmp_path):
    """A resumed engine must run its eager warm-up before capturing (the restored step counter must not skip it)."""
    from gt_b200.ops import native
    from gt_b200.parallel.layers import dist_cross_entropy
    from gt_b200.train.checkpoint import load_checkpoint, save_checkpoint
    from gt_b200.train.engine import TrainEngine
    from gt_b200.train.workloads import exphormer_workload
    dev = _single()

    def build():
        wl = exphormer_workload("exphormer_arxiv", (1, 1), dev, torch.bfloat16, scale_down=32, layers=2, hidden=64, heads=4, dropout=0.1)
        eng = TrainEngine(wl["model"], total_steps=10, warmup=1, use_graph=True, graph_warmup=2)
        x, y, m = wl["x"].to(dev), wl["y"].to(dev), wl["masks"]["train"].to(dev)
        wl["model"].train()
        return wl, eng, (lambda: dist_cross_entropy(wl["model"](x), y, m, wl["n_train"]))

    native.seed_rng(77, dev)
    wl, eng, fn = build()
    ref = [float(eng.train_step(fn)) for _ in range(6)]
    native.seed_rng(77, dev)
    wl, eng, fn = build()
    first = [float(eng.train_step(fn)) for _ in range(3)]
    path = str(tmp_path / "ck.pt")
    save_checkpoint(path, wl["model"], eng, 3)
    wl2, eng2, fn2 = build()
    load_checkpoint(path, wl2["model"], eng2)
    assert eng2.step_count == 3 and eng2._warm_done == 0
    rest = [float(eng2.train_step(fn2)) for _ in range(3)]
    assert eng2._graph is not None                                  # warmed up eagerly (2 steps), then captured
    torch.cuda.synchronize()
    native.check_status(dev)
    got = first + rest
    assert max(abs(a - b) for a, b in zip(got, ref)) < 2e-3, (got, ref)


# ---- several GPUs -------------------------------------------------------------------------------------------------------
MULTI = {
    2: [((2, 1), n) for n in ("plain", "fused", "fused_ln", "fused_nogcn", "fused_gather_proj", "fused_sparse", "pipelined", "streamed", "ring")]
       + [((1, 2), n) for n in ("fused_ln", "fused", "streamed_sync_nocompact")] + [((1, 1, 2), "head"), ((1, 1, 2), "head_gcn")],
    4: [((2, 2), n) for n in ("plain_ln", "fused", "fused_ln", "fused_nogcn", "fused_gather_proj", "fused_sparse", "fused_ckpt", "pipelined",
                              "streamed", "streamed_sync_nocompact")]
       + [((4, 1), "ring"), ((1, 4), "fused_ln"), ((4, 1), "fused_ln"), ((2, 1, 2), "head"), ((1, 2, 2), "head_gcn")],
}
MULTI_VARIANTS = {
    2: [((2, 1), dict(model="unimp")), ((1, 2), dict(model="graphormer")), ((1, 1, 2), dict(model="graphormer", khop=True))],
    4: [((2, 2), dict(model="unimp")), ((2, 2), dict(model="graphormer")), ((2, 1, 2), dict(model="unimp")),
        ((1, 2, 2), dict(model="graphormer", khop=True))],
}


def _multi_worker(rank, world, store, comm, dtype_name):
    import torch.distributed as dist
    from gt_b200.parallel.symm import SymmetricHeap
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"file://{store}", rank=rank, world_size=world, device_id=dev)
    dtype = getattr(torch, dtype_name)
    heap = SymmetricHeap(dev, 512 << 20) if comm == "p2p" else None
    failures = []
    for shape, name in MULTI[world]:
        try:
            _exphormer_case(dev, shape, name, dtype, heap)
            if heap is not None:
                heap.check_symmetric()                        # names the first case after which the ranks' heaps differ
        except Exception as exc:                              # noqa: BLE001  (collected, reported together below)
            failures.append(f"{name} on {shape}: {type(exc).__name__}: {exc}")
    for shape, cfg in MULTI_VARIANTS[world]:
        try:
            _variant_case(dev, shape, cfg, dtype, heap)
        except Exception as exc:                              # noqa: BLE001
            failures.append(f"{cfg} on {shape}: {type(exc).__name__}: {exc}")
    flag = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(flag)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    assert not failures, failures
    assert int(flag) == 0


def _spawn(world, comm, dtype_name):
    import tempfile
    import torch.multiprocessing as mp
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_multi_worker, args=(world, os.path.join(tmp, "store"), comm, dtype_name), nprocs=world, join=True)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
@pytest.mark.parametrize("comm,dtype_name", [("nccl", "float32"), ("p2p", "bfloat16"), ("nccl", "bfloat16")])
def test_layer_kinds_and_variants_two_gpus(comm, dtype_name):
    _spawn(2, comm, dtype_name)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs >= 4 GPUs")
@pytest.mark.parametrize("comm,dtype_name", [("nccl", "float32"), ("p2p", "bfloat16")])
def test_layer_kinds_and_variants_four_gpus(comm, dtype_name):
    _spawn(4, comm, dtype_name)
