"""``bench.py --impl reference``: the unmodified reference (copied to ``baseline/_ref`` by ``install_reference.py``) on the
same synthetic workload, through its own public classes and its stock training path.

What runs: ``gt3d.dist.grid2d.Grid2D`` (``use_axonn=False``), ``gt3d.models.exphormer_dist.DistExphormer`` (fused 2D
layer, LayerNorm, Triton kernels, bf16 wire + bf16 kernel operands, TF32 matmuls: the fastest configuration the
reference documents), ``dist_cross_entropy``, ``allreduce_grads``, ``clip_grad_norm_`` and ``torch.optim.AdamW`` in the
order of ``gt3d/train/train_dist.py:583-627``.  ``train_dist.main()`` itself cannot be called: it loads ogbn-arxiv through
``ogb`` (not installed, no network) or a partition directory without a global token, so the epoch body is restated here
around the reference's classes.  Only the graph generators of this repository are used (input data), none of its models,
kernels or engine.  AxoNN, Plexus and torch_scatter are not installed; ``baseline/shims`` provides the handful of
functions the reference calls from them.
"""
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))


def _unavailable(why):
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    sys.exit(0)


def run_reference(args):
    ref_dir = os.path.join(HERE, "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "gt3d")):
        try:
            from baseline.install_reference import install
            install()
        except SystemExit:
            _unavailable("reference source not present: baseline/_ref missing and the reference checkout is not mounted")
    sys.path.insert(0, os.path.join(HERE, "shims"))
    sys.path.insert(0, ref_dir)
    import torch
    import torch.distributed as dist
    try:
        import triton  # noqa: F401
    except Exception as e:            # the reference's kernels are Triton
        _unavailable(f"triton not importable: {e}")
    if not torch.cuda.is_available():
        _unavailable("no CUDA device on this machine (the reference's kernels and NCCL need one)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    else:
        import tempfile
        dist.init_process_group("nccl", init_method="file://" + os.path.join(tempfile.mkdtemp(), "s"), rank=0, world_size=1)
    rank = dist.get_rank()
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    try:
        from gt3d.dist.grid2d import Grid2D
        from gt3d.dist.layers import allreduce_grads, dist_cross_entropy, set_step
        from gt3d.models.exphormer_dist import DistExphormer, gcn_edges_with_self_loops
        from gt3d.models.exphormer_ref import ExphormerRef
    except Exception as e:
        _unavailable(f"reference import failed: {type(e).__name__}: {e}")

    sys.path.insert(0, os.path.dirname(HERE))
    from bench import REFERENCE_GRIDS, WORKLOAD, ClockSampler
    from gt_b200.data.expander import keyed_expander_edges
    from gt_b200.data.synthetic import virtual_node_edges, workload_graph
    wl = workload_graph(WORKLOAD, seed=0, scale_down=args.scale_down)
    cfg, n = wl["cfg"], wl["n"]
    n_tot = n + 1
    ei = wl["edge_index"]
    exp = keyed_expander_edges(n, 4, seed=0)
    tok = virtual_node_edges(n)[0]
    attn_ei = torch.cat([ei, exp, tok], dim=1)
    attn_et = torch.cat([torch.zeros(ei.shape[1], dtype=torch.long), torch.ones(exp.shape[1], dtype=torch.long),
                         torch.full((tok.shape[1],), 2, dtype=torch.long)])
    n_pad = -(-n_tot // (8 * world)) * (8 * world)
    pd, po = REFERENCE_GRIDS[world]
    grid = Grid2D(pd, po, n_tot, n_pad=n_pad, use_axonn=False).to(dev)
    gcn_blk, _ = grid.local_block(gcn_edges_with_self_loops(ei, n_tot))
    a_blk, a_et = grid.local_block(attn_ei, attn_et)
    torch.manual_seed(0)
    model = DistExphormer(grid, gcn_blk.to(dev), a_blk.to(dev), a_et.to(dev), cfg["features"], cfg["hidden"], cfg["classes"],
                          cfg["layers"], cfg["heads"], dropout=0.1, gnn_dropout=0.1, num_edge_types=3, backend="triton",
                          comm_dtype=torch.bfloat16, fused=True, rs_dtype=torch.bfloat16 if world > 1 else None, norm="ln",
                          kernel_dtype=torch.bfloat16).to(dev)
    for p in model.parameters():
        dist.broadcast(p.data, src=0)
    params = list(model.parameters())
    opt = torch.optim.AdamW(params, lr=1e-3, weight_decay=1e-3)
    x = torch.cat([wl["x"], wl["x"].new_zeros(1, wl["x"].shape[1])])
    y = torch.cat([wl["y"], wl["y"].new_zeros(1)])
    mtr = torch.cat([wl["masks"]["train"], torch.zeros(1, dtype=torch.bool)])
    x_host = grid.take_owned(x).pin_memory()
    y_host = grid.take_owned(y).pin_memory()
    m_host = (grid.take_owned(mtr.to(torch.uint8)).bool() & grid.valid_mask.cpu()).pin_memory()
    x_loc, y_loc, m_loc = x_host.to(dev), y_host.to(dev), m_host.to(dev)
    n_train = int(mtr.sum())
    model.train()
    step_no = [0]

    def step(e2e=False):
        nonlocal x_loc, y_loc, m_loc
        if e2e:
            x_loc = x_host.to(dev, non_blocking=True); y_loc = y_host.to(dev, non_blocking=True); m_loc = m_host.to(dev, non_blocking=True)
        set_step(step_no[0]); step_no[0] += 1
        opt.zero_grad(set_to_none=True)
        logits = model(x_loc)
        loss = dist_cross_entropy(logits, y_loc, m_loc, n_train)
        loss.backward()
        allreduce_grads(params)
        torch.nn.utils.clip_grad_norm_(params, 1.0)
        opt.step()
        return float(loss) if e2e else loss

    try:
        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
    except Exception as e:
        _unavailable(f"reference step failed on this box: {type(e).__name__}: {str(e)[:200]}")

    def timed(fn, steps):
        sampler = ClockSampler(local); sampler.start()
        dist.barrier(); torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.perf_counter(); t0.record()
        for _ in range(steps):
            last = fn()
        t1.record(); torch.cuda.synchronize()
        wall = (time.perf_counter() - w0) * 1e3
        dist.barrier()
        ms = torch.tensor([t0.elapsed_time(t1), wall], device=dev, dtype=torch.float64)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms[0].item() / steps, ms[1].item() / steps, sampler.stop(), last

    ms_dev, _, clocks, loss = timed(lambda: step(False), args.steps)
    _, ms_e2e, clocks2, _ = timed(lambda: step(True), args.steps)
    edges_layers = int(attn_ei.shape[1]) * cfg["layers"]
    if rank == 0:
        h2d = sum(t.numel() * t.element_size() for t in (x_host, y_host, m_host))
        print(json.dumps({
            "impl": "reference",
            "metric": "full-graph train epoch: attention edges/s (E_attn x layers / epoch time), device-timed, max over ranks",
            "value": edges_layers / (ms_dev * 1e-3), "unit": "edges/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_dev, "epoch_s": ms_dev * 1e-3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp32 activations with TF32 matmuls, bf16 attention-kernel operands and bf16 wire (the reference's fastest documented mode)",
            "data": "synthetic (same seeded graph as the gt_b200 arm)",
            "config": {"model": "Exphormer 4L h256 8 heads FFN2x dropout0.1 LayerNorm, reference fused 2D layer, Triton kernels",
                       "nodes": n_tot, "attn_edges": int(attn_ei.shape[1]), "parallelism": "grid %dx%d" % (pd, po),
                       "third_party": "AxoNN / Plexus / torch_scatter replaced by baseline/shims (not installable offline)"},
            "clocks": clocks,
            "e2e": {"value": edges_layers / (ms_e2e * 1e-3), "unit": "edges/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4, "clocks": clocks2},
            "loss": float(loss)}), flush=True)
    from bench import finish
    finish(dist)
