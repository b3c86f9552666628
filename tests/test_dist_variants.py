"""UniMP / Graphormer-node (2D fused and 3D head-parallel) and the TorchGT-style Graphormer vs their single-process
references on gloo CPU ranks (fp64), plus the plain distributed operator and the K/V ring vs the edge-list oracle."""
import pytest
import torch

from dist_utils import grouped_case, run_dist

VARIANTS = {
    "unimp_2x2": dict(model="unimp", grid=(2, 2)),
    "unimp_label_1x2": dict(model="unimp", grid=(1, 2), label=True),
    "unimp_head_2x1x2": dict(model="unimp", grid=(2, 1, 2)),
    "graphormer_2x2": dict(model="graphormer", grid=(2, 2)),
    "graphormer_ckpt_4x1": dict(model="graphormer", grid=(4, 1), checkpoint=True),
    "graphormer_khop_head_1x2x2": dict(model="graphormer", grid=(1, 2, 2), khop=True),
    # the eight-rank layouts of the benchmark configurations
    "unimp_label_head_2x2x2": dict(model="unimp", grid=(2, 2, 2), label=True),
    "graphormer_khop_ckpt_4x2": dict(model="graphormer", grid=(4, 2), khop=True, checkpoint=True),
}


def _variant_worker(rank, world, case, host_heap=False):
    import os, sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from helpers import random_graph
    from gt_b200.data.synthetic import symmetrize, degrees
    from gt_b200.models import gt_variants as gv
    from gt_b200.parallel.grid import make_grid
    from gt_b200.parallel.layers import allreduce_grads, dist_cross_entropy
    cfg = dict(VARIANTS[case])
    n, f, hid, classes, heads = 61, 10, 16, 4, 4
    torch.manual_seed(0)
    ei, _ = random_graph(n, 3, seed=4, hub=True, empty=())
    ei = symmetrize(ei[:, ei[0] != ei[1]], n)
    x = torch.randn(n + 1, f, dtype=torch.float64)
    y = torch.randint(0, classes, (n + 1,))
    mask = torch.rand(n + 1) < 0.6
    mask[n] = False
    grid = make_grid(cfg["grid"], n, n_pad=64)
    if cfg["model"] == "unimp":
        a_ei, a_et = gv.typed_graph_edges(ei, n)
        ref = gv.UniMPRef(f, hid, classes, 2, heads, dropout=0.0, num_classes_label=classes if cfg.get("label") else None).double()
        label_feat = torch.where(torch.rand(n + 1) < 0.5, y, torch.full_like(y, classes)) if cfg.get("label") else None
        out_ref = ref(x[:n], a_ei, label_feat[:n] if label_feat is not None else None)
        kw = dict(num_classes_label=classes if cfg.get("label") else None)
        fw = dict(label_feat=grid.take_owned(label_feat) if label_feat is not None else None)
    else:
        if cfg.get("khop"):
            a_ei, a_et = gv.khop_typed_edges(ei, n)
            nt, tok, outdeg = 3, None, True
            nb = a_ei[:, a_et == 1]
        else:
            a_ei, a_et = gv.graphormer_edges(ei, n)
            nt, tok, outdeg = 4, n, False
            nb = a_ei[:, a_et == 0]
        n_ref = n if cfg.get("khop") else n + 1
        ind, outd = degrees(nb, n_ref)
        ref = gv.GraphormerNodeRef(f, hid, classes, 2, heads, dropout=0.0, max_degree=5, num_edge_types=nt, out_degree=outdeg).double()
        with torch.no_grad():
            ref.attn_bias.normal_()
        out_ref = ref(x[:n_ref], a_ei, a_et, ind, tok, outd if outdeg else None)
        kw = dict(max_degree=5, num_edge_types=nt, out_degree=outdeg, token_row=gv.token_owned_row(grid, n) if tok is not None else None)
        blk_ei, blk_et = grid.local_block(a_ei, a_et)
        d_in, d_out = gv.owned_degrees(grid, blk_ei, blk_et, "cpu", neighbour_type=1 if cfg.get("khop") else 0)
        lo, hi = grid.owned_range()
        nvd = max(min(hi, n_ref) - lo, 0)
        assert (d_in[:nvd] == ind[lo:hi]).all() and (d_out[:nvd] == outd[lo:hi]).all()
        fw = dict(degree_loc=d_in, out_degree_loc=d_out if outdeg else None)
    blk_ei, blk_et = grid.local_block(a_ei, a_et)
    heap = None
    if host_heap:                                           # peer-memory transport between the CPU ranks (shared host memory)
        from gt_b200.parallel.collectives import set_transport
        from gt_b200.parallel.symm_host import HostSymmetricHeap
        heap = HostSymmetricHeap(16 << 20, wait_seconds=60.0, record=True)
        set_transport(heap)
    model = gv.DistGTVariant(grid, blk_ei, blk_et, f, hid, classes, 2, heads, model=cfg["model"], dropout=0.0, backend="torch",
                             checkpoint=cfg.get("checkpoint", False), **kw).double()
    model.load_ref_state_dict(ref.state_dict())
    nm = int(mask.sum())
    loss_ref = torch.nn.functional.cross_entropy(out_ref[mask[:out_ref.shape[0]]], y[:out_ref.shape[0]][mask[:out_ref.shape[0]]], reduction="sum") / nm
    loss_ref.backward()
    model.train()
    out = model(grid.take_owned(x), **fw)
    lo, hi = grid.owned_range()
    nv = max(min(hi, out_ref.shape[0]) - lo, 0)
    assert (out[:nv] - out_ref[lo:lo + nv]).abs().max() < 1e-9
    m_loc = grid.take_owned(mask.to(torch.uint8)).bool()
    dist_cross_entropy(out, grid.take_owned(y), m_loc, nm).backward()
    allreduce_grads(list(model.parameters()))
    rg = dict(ref.named_parameters())
    for name, p in model.named_parameters():
        gr = rg[name].grad
        if gr is None:
            continue
        assert (p.grad - gr).abs().max() < 1e-8 * max(1.0, gr.abs().max().item()), name
    if heap is not None:
        import torch.distributed as dist
        from gt_b200.ops import native
        heap.check_symmetric()
        heap.check_recorded()                               # the recorded accesses are ordered by the recorded barriers
        native.check_status(torch.device("cpu"))
        assert heap.alloc_log[0] > 2, "the case never used the heap"
        dist.barrier()
        set_transport(None)
        heap.close()


def _world_of(case):
    world = 1
    for s in VARIANTS[case]["grid"]:
        world *= s
    return world


@pytest.mark.parametrize("case", list(VARIANTS))
def test_variants_match_reference(case):
    world = _world_of(case)
    grouped_case(_variant_worker, [c for c in VARIANTS if _world_of(c) == world], world, case)


HEAP_VARIANTS = ["unimp_2x2", "unimp_head_2x1x2", "graphormer_2x2", "graphormer_khop_head_1x2x2", "unimp_label_head_2x2x2",
                 "graphormer_khop_ckpt_4x2"]


def _heap_variants_worker(rank, world, cases):
    import torch.distributed as dist
    for case in cases:                                       # one set of processes per world size: a fresh heap and grid per case
        try:
            _variant_worker(rank, world, case, True)
        except Exception as exc:
            raise AssertionError(f"case {case}: {type(exc).__name__}: {exc}") from exc
        dist.barrier()


@pytest.mark.parametrize("world", sorted({_world_of(c) for c in HEAP_VARIANTS}))
def test_variants_match_reference_on_the_host_heap(world):
    """Softmax attention (cross-rank maximum), label inputs, degree embeddings and the head axis with the row collectives on the
    peer-memory transport emulated between the CPU ranks."""
    run_dist(_heap_variants_worker, world, [c for c in HEAP_VARIANTS if _world_of(c) == world], timeout=900)


OPS = {
    "plain_softmax_2x2": dict(grid=(2, 2), op="plain", score="biased", norm="softmax"),
    "plain_clampexp_bf16wire_1x3": dict(grid=(1, 3), op="plain", score="gated", norm="clampexp"),
    "head_softmax_2x1x2": dict(grid=(2, 1, 2), op="head", score="dot", norm="softmax"),
    "ring_kv_3": dict(grid=(3, 1), op="ring_kv"),
    "ring_kv2_4": dict(grid=(4, 1), op="ring_kv", bidir=True),
}


def _op_worker(rank, world, case):
    import os, sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from helpers import random_graph
    from gt_b200.attention import masked_sparse_attention_ref
    from gt_b200.parallel.attention import DistHeadSparseAttention, DistMaskedSparseAttention
    from gt_b200.parallel.grid import make_grid
    from gt_b200.parallel.ring_kv import DistRingAttentionKV
    import torch.distributed as dist
    cfg = OPS[case]
    n, h, d, t = 45, 4, 6, 3
    torch.manual_seed(0)
    ei, et = random_graph(n, 4, seed=8)
    q, k, v = (torch.randn(48, h, d, dtype=torch.float64) for _ in range(3))
    gate, bias = torch.randn(t, h, d, dtype=torch.float64), torch.randn(t, h, dtype=torch.float64)
    w = torch.randn(48, h, d, dtype=torch.float64)
    score, norm = cfg.get("score", "gated"), cfg.get("norm", "clampexp")
    leaves = [x_.clone().requires_grad_() for x_ in (q, k, v, gate, bias)]
    o_ref = masked_sparse_attention_ref(leaves[0], leaves[1], leaves[2], ei, edge_type=et, gate=leaves[3] if score == "gated" else None,
                                        bias=leaves[4] if score == "biased" else None, score=score, norm=norm)
    (o_ref * w).sum().backward()
    grid = make_grid(cfg["grid"], n, n_pad=48)
    b_ei, b_et = grid.local_block(ei, et)
    mine = [grid.take_owned(x_).clone().requires_grad_() for x_ in (q, k, v)]
    g_loc, b_loc = gate.clone().requires_grad_(), bias.clone().requires_grad_()
    if cfg["op"] == "plain":
        op = DistMaskedSparseAttention(grid, (b_ei, b_et), h, d, backend="torch", score=score, norm=norm)
        o = op(*mine, g_loc if score == "gated" else None, b_loc if score == "biased" else None)
    elif cfg["op"] == "head":
        op = DistHeadSparseAttention(grid, (b_ei, b_et), h, d, backend="torch", score=score, norm=norm)
        o = op(*mine, g_loc if score == "gated" else None, b_loc if score == "biased" else None)
    else:
        op = DistRingAttentionKV.from_block(grid, b_ei, b_et, h, d, backend="torch", bidir=cfg.get("bidir", False))
        o = op(*mine, g_loc)
    lo, hi = grid.owned_range()
    assert (o - o_ref[lo:hi]).abs().max() < 1e-10
    (o * w[lo:hi]).sum().backward()
    for a, b in zip(mine, leaves[:3]):
        assert (a.grad - b.grad[lo:hi]).abs().max() < 1e-10
    for a, b, used in ((g_loc, leaves[3], score == "gated"), (b_loc, leaves[4], score == "biased")):
        if used:
            gsum = a.grad.clone()
            dist.all_reduce(gsum)
            assert (gsum - b.grad).abs().max() < 1e-10


def _op_world(case):
    world = 1
    for s in OPS[case]["grid"]:
        world *= s
    return world


@pytest.mark.parametrize("case", list(OPS))
def test_dist_operator_matches_reference(case):
    world = _op_world(case)
    grouped_case(_op_worker, [c for c in OPS if _op_world(c) == world], world, case)


def _torchgt_style_worker(rank, world, fused):
    """``DistGraphormerNode`` (plain and fused routes) against ``GraphormerNode`` with the same weights, fp64, torch backend."""
    import torch.distributed as dist
    from gt_b200.bench.torchgt_batch_bench import torchgt_batch
    from gt_b200.data.synthetic import erdos_renyi, symmetrize
    from gt_b200.models.graphormer_node import DistGraphormerNode, GraphormerNode
    from gt_b200.parallel.grid import Grid2D
    from gt_b200.parallel.layers import allreduce_grads, dist_cross_entropy
    n0, f, hid, classes = 40, 6, 16, 3
    torch.manual_seed(3)
    ei = symmetrize(erdos_renyi(n0, 3, seed=2), n0)
    x, y = torch.randn(n0, f, dtype=torch.float64), torch.randint(0, classes, (n0,))
    xb, yb, eb, n = torchgt_batch(x, y, ei, torch.arange(n0), 30, seed=1)
    ref = GraphormerNode(f, hid, 24, 4, 2, classes, eb, n, dropout=0.0, input_dropout=0.0, backend="torch").double()
    loss_ref = torch.nn.functional.cross_entropy(ref(xb), yb)
    loss_ref.backward()
    grid = Grid2D(2, 1, n) if not fused else Grid2D(1, 2, n)
    b_ei, _ = grid.local_block(eb)
    model = DistGraphormerNode(grid, (b_ei, None), f, hid, 24, 4, 2, classes, dropout=0.0, input_dropout=0.0, backend="torch", fused=fused).double()
    missing = model.load_state_dict(ref.state_dict(), strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    x_loc = grid.take_owned(torch.cat([torch.zeros(1, f, dtype=torch.float64), xb]))
    y_loc = grid.take_owned(torch.cat([torch.zeros(1, dtype=torch.long), yb]))
    mask = grid.valid_mask.clone()
    if grid.owned_range()[0] == 0:
        mask[0] = False
    loss = dist_cross_entropy(model(x_loc), y_loc, mask, n - 1)
    loss.backward()
    params = list(model.parameters())
    allreduce_grads(params)
    tot = loss.detach().clone()
    dist.all_reduce(tot)
    assert abs(float(tot) - float(loss_ref)) < 1e-9
    for (name, p), q in zip(model.named_parameters(), ref.parameters()):
        assert (p.grad - q.grad).abs().max() < 1e-8, name


@pytest.mark.parametrize("fused", [False, True], ids=["plain", "fused"])
def test_torchgt_style_graphormer_matches_single_device(fused):
    run_dist(_torchgt_style_worker, 2, fused)


def _stage_diff_worker(rank, world):
    from gt_b200.utils.stage_diff import main
    rows = main(["--grid", "2", "1", "--fused", "--token", "--token_dense", "--layers", "2"])
    assert [r[0] for r in rows] == ["input stage", "layer 0", "layer 1", "logits"]
    assert all(err < 1e-10 and mag > 0 for _, err, mag in rows), rows


def test_stage_by_stage_diff_tool():
    run_dist(_stage_diff_worker, 2)


def test_state_dict_names_are_the_reference_names_for_every_layer_kind():
    """The checkpoint contract: every distributed model exposes exactly the parameter and buffer names (and shapes) of its reference
    model, whatever layer kind implements it, so a rank-0 ``state_dict()`` is a reference checkpoint and the other way round."""
    from gt_b200.data.expander import random_regular_expander_edges
    from gt_b200.data.synthetic import erdos_renyi, symmetrize
    from gt_b200.models.exphormer_dist import DistExphormer
    from gt_b200.models.exphormer_ref import ExphormerRef, gcn_edges_with_self_loops
    from gt_b200.parallel.grid import make_grid
    from gt_b200.train.engine import init_single_process_group
    init_single_process_group("gloo")
    n, f, hid, classes, heads = 64, 8, 16, 4, 4
    ei = symmetrize(erdos_renyi(n, 4, seed=1), n)
    exp = random_regular_expander_edges(n, 2, seed=1)
    grid = make_grid((1, 1), n, n_pad=64)
    g_blk, _ = grid.local_block(gcn_edges_with_self_loops(ei, n))
    a_ei, a_et = ExphormerRef.build_attention_edges(ei, exp)
    a_blk, a_bt = grid.local_block(a_ei, a_et)
    for norm in ("bn", "ln", "rms"):
        ref = ExphormerRef(f, hid, classes, 2, heads, norm=norm)
        want = {k: tuple(v.shape) for k, v in ref.state_dict().items()}
        for kw in (dict(), dict(fused=True), dict(fused=True, pipeline_sub=2), dict(fused=True, stream_sub=2), dict(fused=True, gather_proj=True),
                   dict(ring=True)):
            model = DistExphormer(grid, g_blk, a_blk, a_bt, f, hid, classes, 2, heads, backend="torch", norm=norm, **kw)
            got = {k: tuple(v.shape) for k, v in model.state_dict().items()}
            assert got == want, (norm, kw, sorted(set(got) ^ set(want)))
            model.load_state_dict(ref.state_dict())            # and the reference checkpoint loads as it is


def test_official_checkpoint_keys_load_into_the_reference_and_distributed_models():
    """A state dict in the key layout of the official implementation (``MultiModel``: ``layers.i.models.1.self_attn.Q.weight`` ...) fills
    the reference model and a distributed model; every tensor arrives where the key map says."""
    import re
    from gt_b200.models import exphormer_ref as er
    from gt_b200.models.exphormer_dist import DistExphormer
    from gt_b200.parallel.grid import make_grid
    from gt_b200.train.engine import init_single_process_group
    init_single_process_group("gloo")
    torch.manual_seed(3)
    src = er.ExphormerRef(8, 16, 4, 2, 4, norm="bn")
    inv_layer = {v: k for k, v in er._LAYER_KEYS.items()}
    inv_norm = {v: k for k, v in er._NORM_PREFIX.items()}
    official = {}
    for key, val in src.state_dict().items():
        if key == "edge_type_emb.weight":
            official["encoder.edge_encoder.encoder.weight"] = val[0:1].clone()
            official["encoder.exp_edge_fixer.exp_edge_attr.weight"] = val[1:2].clone()
        elif key == "pre_lin.weight":
            official["pre_mp.Layer_0.layer.model.weight"] = val.clone()
        elif key.startswith("pre_bn."):
            official["pre_mp.Layer_0.post_layer.0." + key[7:]] = val.clone()
        elif key.startswith("head."):
            official["post_mp.layer_post_mp.model.0.model." + key[5:]] = val.clone()
        else:
            m = re.fullmatch(r"layers\.(\d+)\.(.+)", key)
            rest = m.group(2)
            if rest in inv_layer:
                official[f"layers.{m.group(1)}.{inv_layer[rest]}"] = val.clone()
            else:
                pre = next(p for p in inv_norm if rest.startswith(p))
                official[f"layers.{m.group(1)}.{inv_norm[pre]}{rest[len(pre):]}"] = val.clone()
    assert all(er.official_to_ref_key(k) is not None for k in official) and er.official_to_ref_key("optimizer.state") is None
    dst = er.ExphormerRef(8, 16, 4, 2, 4, norm="bn")
    er.load_official_state_dict(dst, official)
    for k, v in src.state_dict().items():
        assert torch.equal(dst.state_dict()[k], v), k
    n = 32
    from gt_b200.data.synthetic import erdos_renyi, symmetrize
    from gt_b200.data.expander import random_regular_expander_edges
    ei = symmetrize(erdos_renyi(n, 3, seed=1), n)
    grid = make_grid((1, 1), n, n_pad=32)
    a_ei, a_et = er.ExphormerRef.build_attention_edges(ei, random_regular_expander_edges(n, 2, seed=1))
    model = DistExphormer(grid, grid.local_block(er.gcn_edges_with_self_loops(ei, n))[0], *grid.local_block(a_ei, a_et), 8, 16, 4, 2, 4, backend="torch",
                          fused=True)
    er.load_official_state_dict(model, official)
    for k, v in src.state_dict().items():
        assert torch.equal(model.state_dict()[k], v), k
    with pytest.raises(KeyError):
        er.load_official_state_dict(dst, dict(official, **{"encoder.node_encoder.weight": torch.zeros(1)}))
