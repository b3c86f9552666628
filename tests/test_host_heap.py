"""The peer-memory transport between CPU processes (``gt_b200.parallel.symm_host``): the production heap logic on shared host memory,
checked against gloo, on grids with two non-trivial axes."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_dist  # noqa: E402


def _collectives_worker(rank, world, dtype_name):
    import torch.distributed as dist
    from gt_b200.ops import native
    from gt_b200.parallel.grid import make_grid
    from gt_b200.parallel.sparse_comm import SparseRowPlan
    from gt_b200.parallel.symm_host import HostSymmetricHeap
    dtype = getattr(torch, dtype_name)
    tol = dict(float64=1e-12, float32=1e-5, bfloat16=5e-2)[dtype_name]
    grid = make_grid((2, 2), 64, n_pad=64)
    heap = HostSymmetricHeap(8 << 20, wait_seconds=30.0, record=True)
    g = torch.Generator().manual_seed(100 + rank)
    try:
        for rep in range(3):                                 # three rounds: every staging copy is reused
            heap.begin_step()
            for group in (grid.row_group, grid.col_group, None):
                size = dist.get_world_size(group)
                me = dist.get_rank(group)
                x = torch.randn(24, 16, generator=g).to(dtype)
                ref = [torch.empty_like(x) for _ in range(size)]
                dist.all_gather(ref, x, group=group)
                assert torch.equal(heap.all_gather(x, group), torch.cat(ref)), "all_gather"
                y = torch.randn(size * 8, 16, generator=g).to(dtype)
                tot = y.double().clone()
                dist.all_reduce(tot, group=group)
                got = heap.reduce_scatter(y, group)
                assert (got.double() - tot[me * 8:(me + 1) * 8]).abs().max() < tol * size, "reduce_scatter"
                z = torch.randn(40, generator=g).to(dtype)
                tot = z.double().clone()
                dist.all_reduce(tot, group=group)
                assert (heap.all_reduce(z, torch.empty_like(z), group=group).double() - tot).abs().max() < tol * size, "all_reduce"
                h = torch.randn(6, 2 * size, 8, generator=g).to(dtype)            # Ulysses all-to-all, there and back
                t = heap.rows_to_heads(h, group)
                send = h.view(6, size, 2, 8).transpose(0, 1).contiguous()
                recv = torch.empty_like(send)
                dist.all_to_all_single(recv, send, group=group)
                assert torch.equal(t, recv.view(size * 6, 2, 8)), "rows_to_heads"
                assert torch.equal(heap.heads_to_rows(t, group), h), "heads_to_rows"
            # sparse plans whose need sets differ between the two row groups (3 rows against 29) and between the members of a group
            per = grid.n_row_block // 2
            n_need = (3 if grid.r == 0 else 29) + grid.c
            need = torch.randperm(2 * per, generator=torch.Generator().manual_seed(7 + rank))[:n_need].sort().values
            plans = {t: SparseRowPlan(grid.row_group, per, need, "row", t, heap if t == "pull" else None) for t in ("a2a", "pull")}
            x = torch.randn(per, 16, generator=g).to(dtype)
            assert torch.equal(plans["pull"].gather(x), plans["a2a"].gather(x)), "sparse gather"
            y = torch.randn(n_need, 16, generator=g).to(dtype)
            a, b = plans["pull"].reduce_scatter(y), plans["a2a"].reduce_scatter(y)
            assert (a.double() - b.double()).abs().max() < tol * 2, "sparse reduce_scatter"
            # a collective of the COLUMN group right after the row groups grew their heaps: the offsets must still agree
            x = torch.randn(8, 16, generator=g).to(dtype)
            ref = [torch.empty_like(x) for _ in range(2)]
            dist.all_gather(ref, x, group=grid.col_group)
            assert torch.equal(heap.all_gather(x, grid.col_group), torch.cat(ref)), "all_gather after the sparse plans"
            heap.check_symmetric()
        if dtype == torch.float32:                           # two-shot all-reduce of named heap tensors over epoch channels
            n = 1000
            src = heap.empty(n, torch.float32, "grads")
            heap.empty(n, torch.float32, "grads_sum")
            for rep in range(3):
                src.copy_(torch.arange(n, dtype=torch.float32) * (rank + 1) + rep)
                heap.all_reduce_two_shot("grads", "grads_sum", n)
                want = torch.arange(n, dtype=torch.float32) * sum(range(1, world + 1)) + rep * world
                assert torch.equal(heap.view(heap.named["grads_sum"][0], (n,), torch.float32), want), "two-shot all-reduce"
            heap.check_symmetric()
        native.check_status(torch.device("cpu"))
        rep = heap.check_recorded()                          # every recorded access is ordered by the recorded signals and waits
        assert rep.n_ops > 500
    finally:
        dist.barrier()
        heap.close()


@pytest.mark.parametrize("dtype_name", ["float64", "float32", "bfloat16"])
def test_heap_collectives_match_gloo_on_a_2x2_grid(dtype_name):
    run_dist(_collectives_worker, 4, dtype_name)


def _expiry_worker(rank, world):
    import torch.distributed as dist
    from gt_b200.ops import native
    from gt_b200.parallel.symm_host import HostSymmetricHeap
    heap = HostSymmetricHeap(1 << 20, wait_seconds=2.0)
    ctx = heap.ctx(None)
    dist.barrier()
    if rank != 1:                                            # rank 1 never arrives: the others give up after the limit and say who
        ctx.barrier()
        with pytest.raises(RuntimeError, match="code 101"):
            native.check_status(torch.device("cpu"))
        native.check_status(torch.device("cpu"))             # the word was cleared; the process carries on
    dist.barrier()
    heap.close()


def test_a_silent_rank_expires_the_barrier_with_its_index():
    run_dist(_expiry_worker, 3)


FAMILIES = ("x_col", "x_row", "pay", "dpay", "dx_col", "dx_row")


def _compare_with_protocol_model(log, model, grid, rank):
    """The sequence of writes, reads, signals and waits that the operator made on shared memory equals the program of this rank in
    ``gt_b200.parallel.protocol_model`` (the input of the happens-before check): the model describes the code."""
    from gt_b200.parallel import protocol_model as pm
    comms = [layer._fb_comm for layer in model.layers]
    chan = {}
    for li, c in enumerate(comms):
        for fam in FAMILIES:
            ch = getattr(c, fam)
            chan[ch.off] = (fam + str(li), ch.ctx.ranks)
    bufs = []
    for ctx in (comms[0].col, comms[0].row):
        for key, (off, nbytes) in ctx.buffers.items():
            if isinstance(key, tuple) and isinstance(key[0], str) and key[0].startswith("fb_"):
                slots = ctx.size if key[0] in ("fb_pay", "fb_dxc", "fb_dxr") else 1
                bufs.append((off, nbytes, key[0], key[1], slots))

    def locate(off):
        for base, nbytes, kind, copy, slots in bufs:
            if base <= off < base + nbytes:
                return kind, copy, slots, (off - base) // (nbytes // slots)
        return None

    got, since_signal = [], set()
    for ev in log:
        if ev[0] == "signal":
            if ev[1] in chan:
                got.append(("signal", chan[ev[1]][0]))
                since_signal = set()
        elif ev[0] == "wait":
            if ev[1] in chan:
                name, ranks = chan[ev[1]]
                got.append(("wait", name, ranks[ev[2]]))
        elif ev[0] in ("view", "write", "read"):
            at = locate(ev[2])
            if at is None:
                continue
            kind, copy, slots, slot = at
            if ev[0] == "view":
                if kind == "fb_x" and ev[1] == rank:         # x is copied into its staging buffer through a tensor view
                    got.append(("write", rank, kind, copy, None))
                continue
            if ev[0] == "read" and slots > 1:                # the owner reads all slots of the buffer in one kernel
                got.extend(("read", ev[1], kind, copy, s_) for s_ in range(slots))
                continue
            item = (ev[0], ev[1], kind, copy, slot if slots > 1 else None)
            if ev[0] == "write":
                if item in since_signal:                     # attention rows and aggregation rows go into the same slot
                    continue
                since_signal.add(item)
            got.append(item)
    want = []
    prog = pm.fused_step_trace(grid.p_rows, grid.p_cols, len(comms), steps=2).prog[rank]
    for op, a, b, _, _ in prog:
        if op in ("write", "read"):
            if len(b) > 1 and isinstance(b[1], str) and b[1].startswith("fb_"):
                want.append((op, a, b[1], b[2], b[3] if len(b) > 3 else None))
        elif op == "signal":
            if a[0].rstrip("0123456789") in FAMILIES:
                want.append(("signal", a[0]))
        elif a[0].rstrip("0123456789") in FAMILIES:
            want.append(("wait", a[0], b))
    assert len(got) == len(want), (len(got), len(want))
    for i, (g_, w_) in enumerate(zip(got, want)):
        assert g_ == w_, (i, g_, w_)


def _fused_worker(rank, world, grid_shape, cfg):
    """The fused 2D layer as ONE operator with its collectives inside the (emulated) kernels, bf16, against the fp64 reference model:
    logits, loss and every parameter gradient, two steps in a row (every staging copy and channel is reused)."""
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import torch.distributed as dist
    from helpers import random_graph
    from test_gpu_parity import TOL, _grad_err, _grad_floor
    from gt_b200.data.expander import random_regular_expander_edges
    from gt_b200.models.exphormer_dist import DistExphormer
    from gt_b200.models.exphormer_ref import ExphormerRef, gcn_edges_with_self_loops
    from gt_b200.ops import native
    from gt_b200.parallel import fused_layer
    from gt_b200.parallel.collectives import set_transport
    from gt_b200.parallel.grid import make_grid
    from gt_b200.parallel.layers import dist_cross_entropy, set_step
    from gt_b200.parallel.symm_host import HostSymmetricHeap
    from gt_b200.train.engine import TrainEngine
    cfg = dict(cfg)
    token = cfg.pop("token", False)                           # a global token, computed as dense terms outside the operator
    n, f, hid, classes, heads = 500 - (1 if token else 0), 16, 64, 8, 4
    torch.manual_seed(0)
    ei, _ = random_graph(n, 4, seed=3, hub=True, empty=())
    ei = ei[:, ei[0] != ei[1]]
    exp = random_regular_expander_edges(n, 3, seed=1)
    tok = None
    if token:
        from gt_b200.data.synthetic import virtual_node_edges
        tok = virtual_node_edges(n)[0]
        cfg.update(token_node=n, num_edge_types=3)
        n += 1
    x = torch.randn(n, f, dtype=torch.float64)
    y = torch.randint(0, classes, (n,))
    mask = torch.rand(n) < 0.6
    with_gcn = cfg.get("with_gcn", True)
    ref = ExphormerRef(f, hid, classes, 2, heads, dropout=0.0, gnn_dropout=0.0, with_gcn=with_gcn, norm="ln", num_edge_types=3 if token else 2).double()
    n_pad = -(-n // (16 * world)) * (16 * world)
    grid = make_grid(grid_shape, n, n_pad=n_pad)
    gcn_blk, _ = grid.local_block(gcn_edges_with_self_loops(ei, n))
    attn_ei, attn_et = ExphormerRef.build_attention_edges(ei, exp)
    a_blk, a_et = grid.local_block(attn_ei, attn_et)
    heap = HostSymmetricHeap(32 << 20, wait_seconds=60.0, record=True)
    set_transport(heap)
    bf = torch.bfloat16
    model = DistExphormer(grid, gcn_blk, a_blk, a_et, f, hid, classes, 2, heads, dropout=0.0, gnn_dropout=0.0, backend="torch", fused=True,
                          norm="ln", comm_dtype=bf, rs_dtype=bf, kernel_dtype=bf, heap=heap, **cfg)
    model.load_ref_state_dict(ref.state_dict())
    eng = TrainEngine(model, heap=heap)
    # as on GPUs: the operator reads K | V | message | Q from the engine's stacked bf16 shadow and adds their gradients into its flat buffer
    assert all(layer._w_stack is not None and layer._w_stack[1] is not None for layer in model.layers)
    calls = {"n": 0}
    real = fused_layer._FusedBranch.apply

    def counted(*a):
        calls["n"] += 1
        return real(*a)
    fused_layer._FusedBranch.apply = counted
    set_step(0)
    ref.train(); model.train()
    out_ref = ref(x, ei, exp, tok)
    loss_ref = torch.nn.functional.cross_entropy(out_ref[mask], y[mask], reduction="sum") / int(mask.sum())
    loss_ref.backward()
    ref_grads = dict(ref.named_parameters())
    floor = _grad_floor(ref_grads)
    tol_f, tol_g = TOL[bf]
    lo, hi = grid.owned_range()
    nv = max(min(hi, n) - lo, 0)
    failures = []
    del native.ext().log[:]                                   # from here: what the operator does to shared memory, in order
    for step in range(2):
        dist.barrier()
        heap.begin_step()
        eng.flat_g.zero_()
        out = model(grid.take_owned(x).to(bf))
        err = (out[:nv].double() - out_ref[lo:lo + nv]).abs().max().item() / out_ref.abs().max().item() if nv else 0.0
        m_loc = grid.take_owned(mask.to(torch.uint8)).bool() & grid.valid_mask
        loss = dist_cross_entropy(out, grid.take_owned(y), m_loc, int(mask.sum()))
        loss.backward()
        tot = loss.detach().float().clone()
        dist.all_reduce(tot)
        g = eng._reduce_grads()                               # the two-shot all-reduce of the heap
        if err >= tol_f:
            failures.append(("logits", step, err))
        if abs(tot.item() - loss_ref.item()) >= tol_f * max(1.0, abs(loss_ref.item())) * 4:
            failures.append(("loss", step, tot.item(), loss_ref.item()))
        for pname, p in model.named_parameters():
            gr = ref_grads[pname].grad
            if gr is None:
                continue
            off = eng.offsets[id(p)]
            e_ = _grad_err(g[off:off + p.numel()].view_as(p), gr, floor)
            if e_ >= tol_g:
                failures.append((pname, step, e_))
    native.check_status(torch.device("cpu"))
    heap.check_symmetric()
    fused_layer._FusedBranch.apply = real
    assert calls["n"] == 2 * 2, calls                         # two layers, two steps: the operator ran, not the op-by-op fallback
    assert not failures, failures
    if world > 1:
        _compare_with_protocol_model(native.ext().log, model, grid, rank)
        heap.check_recorded()                                 # and the recorded run itself passes the happens-before check
    dist.barrier()
    set_transport(None)
    heap.close()


FUSED_GRIDS = [((2, 2), {}), ((2, 1), {}), ((1, 2), {}), ((4, 2), {}), ((2, 4), {}), ((2, 2), dict(with_gcn=False)), ((3, 2), {}),
               ((2, 2), dict(token=True)), ((4, 2), dict(token=True)), ((1, 1), {}), ((1, 1), dict(token=True))]


def _fused_cases_worker(rank, world, cases):
    import torch.distributed as dist
    for grid_shape, cfg in cases:                            # one set of processes per world size: a fresh heap, grid and model per case
        try:
            _fused_worker(rank, world, grid_shape, cfg)
        except Exception as exc:
            raise AssertionError(f"grid {grid_shape} {cfg}: {type(exc).__name__}: {exc}") from exc
        dist.barrier()


@pytest.mark.parametrize("world", sorted({g[0] * g[1] for g, _ in FUSED_GRIDS}))
def test_fused_operator_with_in_kernel_collectives_between_cpu_ranks(world):
    run_dist(_fused_cases_worker, world, [(g, c) for g, c in FUSED_GRIDS if g[0] * g[1] == world], timeout=900)


def _single_copy_worker(rank, world):
    """Negative control of the recorded check: with ONE staging copy per kind a rank may rewrite its buffer while a peer still reads the
    previous contents.  Whether that corrupts data depends on timing; the happens-before check of the recorded run reports it always."""
    import torch.distributed as dist
    from gt_b200.parallel import symm
    from gt_b200.parallel.symm_host import HostSymmetricHeap
    orig = symm.GroupContext.staging

    def one_copy(self, nbytes, kind):
        self.kind_count[kind] = 0
        return orig(self, nbytes, kind)
    heap = HostSymmetricHeap(4 << 20, wait_seconds=30.0, record=True)
    try:
        x = torch.randn(16, 8)
        for _ in range(4):
            heap.all_gather(x, None)
        heap.check_recorded()                                # two copies: ordered
        symm.GroupContext.staging = one_copy
        for _ in range(4):
            heap.all_gather(x, None)
        with pytest.raises(RuntimeError, match="write-while-read|read-before-write"):
            heap.check_recorded()
    finally:
        symm.GroupContext.staging = orig
        dist.barrier()
        heap.close()


def test_recorded_check_reports_single_buffering():
    run_dist(_single_copy_worker, 3)


def _train_steps_worker(rank, world, grid_shape):
    """Whole training steps through ``TrainEngine.train_step`` with the fused operator on the host transport: the loss falls, no wait
    expires, and the replicated parameters stay bit-identical on all ranks (every rank gets the same reduced gradient)."""
    import torch.distributed as dist
    from gt_b200.ops import native
    from gt_b200.parallel.collectives import set_transport
    from gt_b200.parallel.layers import dist_cross_entropy
    from gt_b200.parallel.symm_host import HostSymmetricHeap
    from gt_b200.train.engine import TrainEngine
    from gt_b200.train.workloads import exphormer_workload
    heap = HostSymmetricHeap(64 << 20, wait_seconds=60.0, record=True)
    set_transport(heap)
    wl = exphormer_workload("cpu_small", grid_shape, "cpu", torch.bfloat16, seed=0, heap=heap, scale_down=4, dropout=0.0, layers=2, hidden=32, heads=4,
                            kernel_dtype=torch.bfloat16, comm_dtype=torch.bfloat16, rs_dtype=torch.bfloat16)
    model = wl["model"]
    for p in model.parameters():
        dist.broadcast(p.data, src=0)
    eng = TrainEngine(model, lr=2e-2, weight_decay=0.0, total_steps=12, warmup=1, heap=heap)
    assert all(layer._w_stack is not None for layer in model.layers)
    x, y, m = wl["x"], wl["y"], wl["masks"]["train"]
    from gt_b200.parallel import fused_layer
    calls, real = {"n": 0}, fused_layer._FusedBranch.apply

    def counted(*a):
        calls["n"] += 1
        return real(*a)
    fused_layer._FusedBranch.apply = counted
    losses = []
    for _ in range(6):
        loss = eng.train_step(lambda: dist_cross_entropy(model(x), y, m, wl["n_train"]))
        tot = loss.detach().float().clone()
        dist.all_reduce(tot)
        losses.append(tot.item())
    fused_layer._FusedBranch.apply = real
    native.check_status(torch.device("cpu"))
    assert calls["n"] == 6 * 2, calls                         # the operator ran in every layer of every step
    assert all(torch.isfinite(torch.tensor(losses))) and losses[-1] < losses[0] - 0.05, losses
    flat = [torch.empty_like(eng.flat_p) for _ in range(world)]
    dist.all_gather(flat, eng.flat_p)
    assert all(torch.equal(flat[0], f) for f in flat[1:]), "replicated parameters differ between ranks"
    assert torch.equal(eng.flat_p_bf16.float(), eng.flat_p.to(torch.bfloat16).float())          # the shadow follows the optimizer
    heap.check_symmetric()
    heap.check_recorded()
    dist.barrier()
    set_transport(None)
    heap.close()


def test_training_steps_with_the_fused_operator_between_cpu_ranks():
    run_dist(_train_steps_worker, 4, (2, 2))


def test_emulated_entry_points_keep_the_signatures_of_the_native_binding():
    """Drift guard: every entry point that the host emulation restates takes as many arguments as the function of the same name in the
    native module (whose Python-visible signatures pybind11 writes into the docstrings).  A change of a binding that is not mirrored
    here would otherwise only show up as a TypeError in some emulated run."""
    import inspect
    from gt_b200 import build_ext
    from gt_b200.parallel.symm_host import HostExt
    mod = build_ext.load_prebuilt()
    if mod is None:
        pytest.skip("the native module is not built here")
    checked = 0
    for name, fn in inspect.getmembers(HostExt, predicate=inspect.isfunction):
        if name.startswith("_"):
            continue
        assert hasattr(mod, name), f"{name} is emulated but the native module has no such entry point"
        doc = getattr(mod, name).__doc__.splitlines()[0]
        inner = doc[doc.index("(") + 1:doc.rindex(")")]
        depth, n = 0, 1 if inner.strip() else 0
        for ch in inner:
            depth += ch in "[("
            depth -= ch in "])"
            n += ch == "," and depth == 0
        params = [p for p in inspect.signature(fn).parameters if p != "self"]
        assert n == len(params), (name, doc, params)
        checked += 1
    assert checked >= 30


def _refuse_worker(rank, world):
    """A collective of the heap over a group that crosses (pretended) machines is refused on the host; it never reaches a kernel."""
    import torch.distributed as dist
    os.environ["GT_HOSTNAME"] = "node%d" % (rank // 2)
    from gt_b200.parallel.symm_host import HostSymmetricHeap
    try:
        heap = HostSymmetricHeap(1 << 20)
        assert not heap.group_is_local(None) and heap.peer_base[(rank + 2) % 4] == 0 and heap.peer_base[rank ^ 1] != 0
        pair = [dist.new_group([0, 1]), dist.new_group([2, 3])][rank // 2]
        assert heap.group_is_local(pair)
        x = torch.full((8, 8), float(rank))
        assert torch.equal(heap.all_gather(x, pair)[8:], torch.full((8, 8), float(rank | 1)))
        with pytest.raises(RuntimeError, match="crosses machines"):
            heap.all_gather(x, None)
        dist.barrier()
        heap.close()
    finally:
        os.environ.pop("GT_HOSTNAME", None)


def test_heap_refuses_groups_that_cross_machines():
    run_dist(_refuse_worker, 4)


def test_edge_rows_from_a_segment_plan_match_the_csr_rows():
    """The host kernels recover the row (or column) of every entry from a pass's segment list: hub rows cut into several segments,
    empty rows, the longest-first order of the segments and the transposed (column) plan included."""
    from gt_b200.attention.backend_cuda import _plan_list
    from gt_b200.attention.csr import BlockCSR
    from gt_b200.parallel.fused_host import _edge_rows
    g = torch.Generator().manual_seed(5)
    n_rows, n_cols = 300, 257
    dst = torch.cat([torch.randint(0, n_rows, (2000,), generator=g), torch.full((900,), 7), torch.full((40,), 11)])      # rows 7 and 11 are hubs
    src = torch.randint(0, n_cols, (dst.numel(),), generator=g)
    ei = torch.unique(torch.stack([src, dst]), dim=1)
    blk = BlockCSR.from_edges(ei, n_rows, n_cols, torch.zeros(ei.shape[1], dtype=torch.long))
    for seg in (16, 64, 512):
        plan = blk.row_plan(seg)
        assert plan.num_segments > n_rows // 2 and int((plan.seg_end - plan.seg_beg).max()) <= seg
        assert torch.equal(_edge_rows(_plan_list(plan), blk.num_edges), blk.rows().long())
        _, rowidx, _, pos, _ = blk.csc()
        cols = _edge_rows(_plan_list(blk.col_plan(seg)), blk.num_edges)
        assert torch.equal(cols, blk.col.long()[pos.long()])                # the column of every CSC entry
        assert torch.equal(rowidx.long(), blk.rows().long()[pos.long()])


def test_every_python_call_into_the_native_module_passes_the_bound_number_of_arguments():
    """Static drift guard: the bindings declare no default arguments, so every ``ext().f(...)`` / ``e.f(...)`` call in the package must
    pass exactly as many positional arguments as the bound function takes (a wrong count would only fail when that line runs on a GPU)."""
    import ast
    import glob
    from gt_b200 import build_ext
    mod = build_ext.load_prebuilt()
    if mod is None:
        pytest.skip("the native module is not built here")

    def arity(fn):
        doc = fn.__doc__.splitlines()[0]
        inner = doc[doc.index("(") + 1:doc.rindex(")")]
        depth, n = 0, 1 if inner.strip() else 0
        for ch in inner:
            depth += ch in "[("
            depth -= ch in "])"
            n += ch == "," and depth == 0
        return n
    bound = {name: arity(getattr(mod, name)) for name in dir(mod) if not name.startswith("_") and callable(getattr(mod, name))}

    def is_ext(node):                                        # e, ext(), native.ext(), self.ext() ...
        if isinstance(node, ast.Name):
            return node.id == "e"
        if isinstance(node, ast.Call):
            f = node.func
            return (isinstance(f, ast.Name) and f.id == "ext") or (isinstance(f, ast.Attribute) and f.attr == "ext")
        return False
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    checked, wrong = 0, []
    files = glob.glob(os.path.join(root, "gt_b200", "**", "*.py"), recursive=True) + glob.glob(os.path.join(root, "tests", "*.py")) \
        + [os.path.join(root, "bench.py")]
    for path in files:
        tree = ast.parse(open(path).read())
        for node in ast.walk(tree):
            if isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and node.func.attr in bound and is_ext(node.func.value):
                if any(isinstance(a, ast.Starred) for a in node.args):
                    continue
                checked += 1
                if node.keywords or len(node.args) != bound[node.func.attr]:
                    wrong.append((os.path.relpath(path, root), node.lineno, node.func.attr, len(node.args), bound[node.func.attr]))
    assert not wrong, wrong
    assert checked >= 80, checked
