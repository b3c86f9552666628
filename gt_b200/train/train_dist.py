"""Distributed full-graph trainer (one process per GPU, or CPU ranks on gloo).

    torchrun --nproc-per-node 4 -m gt_b200.train.train_dist --grid 2 2 --fused --synthetic exphormer_arxiv --bf16
    torchrun --nproc-per-node 8 -m gt_b200.train.train_dist --grid 2 2 2 --no_gcn --data /data/products_p16
    python -m gt_b200.train.train_dist --grid 1 1 --synthetic cpu_small --epochs 20          (single process)

One epoch is one full-graph step: forward, masked cross-entropy, backward, gradient all-reduce, global-norm clipping,
AdamW, cosine schedule.  The flag set and the log grammar (``data:``, ``[mem]``, ``epoch ...``, ``FINAL``, ``STEADY
ms_per_epoch= peak_gb=``) follow the reference trainer (``gt3d/gt3d/train/train_dist.py:329-381, 501-510, 648-679``) so
scripts and parsers written for it keep working; epoch times are measured on the device (CUDA events, max over ranks)
instead of the host wall clock.  Additions: ``--synthetic``, ``--bf16``, ``--cuda_graph``, ``--comm p2p`` (peer-memory
kernels instead of NCCL), ``--save`` / ``--resume`` (checkpoints).
"""
import argparse
import contextlib
import os
import time

import torch
import torch.distributed as dist


def build_parser():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    a = ap.add_argument
    a("--grid", type=int, nargs="+", default=[1, 1], help="P_d P_o (2D block grid) or P_d P_o P_i (head axis: P_i divides --heads)")
    a("--grid_layout", default="row_major", choices=["row_major", "col_major"])
    a("--grid_auto", action="store_true", help="pick the 2D grid with the performance / memory model")
    a("--head_auto", action="store_true", help="pick among 2D fused grids and 3D head grids with the model")
    a("--backend", default=None, choices=["torch", "cuda", "triton"], help="attention backend (default: cuda on GPUs, torch on CPU; 'triton' is an alias of 'cuda')")
    a("--model", default="exphormer", choices=["exphormer", "unimp", "graphormer"])
    a("--epochs", type=int, default=100)
    a("--warmup", type=int, default=5)
    a("--hidden", type=int, default=None)
    a("--heads", type=int, default=None)
    a("--layers", type=int, default=None)
    a("--dropout", type=float, default=0.3)
    a("--lr", type=float, default=1e-3)
    a("--weight_decay", type=float, default=1e-3)
    a("--exp_deg", type=int, default=3)
    a("--seed", type=int, default=0)
    a("--eval_every", type=int, default=1)
    a("--timing_epochs", type=int, default=0, help="run this many epochs, evaluate only at the end")
    a("--data", default=None, help="partition directory (gt_b200.data.partition or Plexus layout)")
    a("--synthetic", default=None, help="synthetic workload name (gt_b200.data.synthetic.WORKLOADS); default cpu_small")
    a("--scale_down", type=int, default=1)
    a("--eval_only", action="store_true",
      help="with --resume: load the checkpoint, evaluate train / validation / test accuracy once (eval mode, no gradient) and exit")
    a("--metrics_jsonl", default=None, metavar="FILE",
      help="rank 0 appends one JSON object per evaluated epoch (epoch, loss, accuracies, device ms of the epoch, best so far)")
    a("--predict_out", default=None, metavar="FILE",
      help="with --eval_only: rank 0 writes {'pred': int64 [N] predicted classes in node order, 'num_nodes': N} to FILE")
    a("--heartbeat", type=float, default=0.0, metavar="SECONDS",
      help="host-side failure detection: every rank bumps a counter in the job's store once per epoch and checks its peers' before "
           "launching the step; a peer that announced a failure or was silent for SECONDS ends the run with PeerFailure (0 = off)")
    a("--stream_gen", action="store_true",
      help="(--synthetic exphormer_rmat26) build every rank's blocks from streamed edge chunks: no rank holds the global graph")
    a("--virtual_node", action="store_true", help="(exphormer) add one global token connected to every node (edge type 2)")
    a("--token_dense", action="store_true",
      help="(--virtual_node, fused / pipelined layers) keep the token's 2 n edges out of the sparse blocks and compute its row and column as "
           "dense terms on the owned rows plus one small all-reduce: no rank carries the token's row or column")
    a("--graph_name", default=None)
    # layer kind
    a("--fused", action="store_true", help="fused-communication layer: gather x once, one reduce-scatter")
    a("--pipeline_sub", type=int, default=1)
    a("--stream_sub", type=int, default=1)
    a("--ring", action="store_true")
    a("--gather_proj", action="store_true")
    a("--no_gcn", action="store_true")
    a("--no_attn", action="store_true")
    a("--stream_overlap", action="store_true")
    a("--no_stream_overlap", action="store_true")
    a("--no_stream_compact", action="store_true")
    a("--checkpoint", action="store_true", help="activation checkpointing per layer")
    a("--auto_ckpt", action="store_true")
    a("--compile", action="store_true", help="accepted for compatibility; the step is captured in a CUDA graph instead (--cuda_graph)")
    # numerics
    a("--bf16", action="store_true", help="bf16 activations / kernels with fp32 master weights")
    a("--comm_bf16", action="store_true")
    a("--rs_bf16", action="store_true")
    a("--kernel_bf16", action="store_true")
    a("--tf32_matmul", action="store_true")
    a("--no_tf32_matmul", action="store_true")
    a("--norm", default="bn", choices=["bn", "ln", "rms"])
    a("--label_input", action="store_true")
    a("--label_rate", type=float, default=0.5)
    a("--max_degree", type=int, default=64)
    a("--ffn_mult", type=int, default=2)
    a("--khop", action="store_true", help="(graphormer) 2-hop mask with shortest-path-bucket bias and in/out-degree embeddings")
    # communication
    a("--comm", default="nccl", choices=["nccl", "p2p"],
      help="grid collectives: NCCL (gloo on CPU ranks) or the peer-memory transport (symmetric heap; between CPU ranks an emulation over shared host memory)")
    a("--heap_mb", type=int, default=2048)
    a("--check_protocol", action="store_true",
      help="(--comm p2p between CPU ranks) record every access to shared memory with the signals, barriers and waits around it, and run the "
           "happens-before check on the recorded run at the end: a race check of this configuration's peer-memory protocol without GPUs")
    a("--nccl_tune", default="auto", choices=["auto", "on", "off"])
    a("--sparse_comm", action="store_true")
    a("--sparse_threshold", type=float, default=None)
    a("--sparse_threshold_row", type=float, default=None)
    # run control / observability
    a("--cuda_graph", action="store_true", help="capture the whole training step in a CUDA graph")
    a("--save", default=None, help="write a checkpoint here (every --save_every epochs and at the end)")
    a("--save_every", type=int, default=0)
    a("--resume", default=None)
    a("--profile", action="store_true")
    a("--timers", action="store_true")
    a("--coll_stats", action="store_true")
    a("--saved_census", action="store_true")
    return ap


def parse_with_config(ap, argv=None):
    """``--config FILE`` (YAML or JSON mapping of flag names to values) supplies defaults; flags on the command line win.
    Unknown keys are an error, so a misspelt option does not pass silently."""
    pre = argparse.ArgumentParser(add_help=False)
    pre.add_argument("--config", default=None)
    known, _ = pre.parse_known_args(argv)
    ap.add_argument("--config", default=None, metavar="FILE", help="YAML / JSON file with default values for the flags above")
    if known.config:
        with open(known.config) as f:
            text = f.read()
        if known.config.endswith(".json"):
            import json
            cfg = json.loads(text)
        else:
            import yaml
            cfg = yaml.safe_load(text) or {}
        if not isinstance(cfg, dict):
            raise SystemExit(f"--config {known.config}: expected a mapping of flag names to values")
        dests = {a.dest for a in ap._actions}
        cfg = {str(k).lstrip("-").replace("-", "_"): v for k, v in cfg.items()}
        unknown = sorted(set(cfg) - dests)
        if unknown:
            raise SystemExit(f"--config {known.config}: unknown options {unknown}")
        ap.set_defaults(**cfg)
    return ap.parse_args(argv)


def validate(args):
    args.stream_overlap = not args.no_stream_overlap
    if args.backend == "triton":
        args.backend = "cuda"
    if args.timing_epochs > 0:
        args.epochs = args.timing_epochs
        args.eval_every = args.timing_epochs
    if len(args.grid) not in (2, 3):
        raise SystemExit("--grid takes P_d P_o or P_d P_o P_i")
    head = len(args.grid) == 3
    if args.ring and (args.grid[1] != 1 or args.grid_auto):
        raise SystemExit("--ring needs --grid P 1")
    if head and (args.fused or args.ring or args.gather_proj or max(args.pipeline_sub, args.stream_sub) > 1 or args.grid_auto):
        raise SystemExit("the head grid has its own layer: no --fused / --ring / --gather_proj / --pipeline_sub / --stream_sub / --grid_auto")
    if args.sparse_comm and args.model != "exphormer":
        raise SystemExit("--sparse_comm is implemented for the Exphormer layers")
    if args.check_protocol and (args.comm != "p2p" or torch.cuda.is_available()):
        raise SystemExit("--check_protocol records the host emulation of the peer-memory transport: CPU ranks with --comm p2p")
    if args.token_dense and not (args.virtual_node and args.model == "exphormer" and args.fused and not head and not args.ring
                                 and args.stream_sub <= 1 and args.data is None and not args.stream_gen):
        raise SystemExit("--token_dense needs --virtual_node with the fused or pipelined Exphormer layer on a synthetic graph")
    return head


def init_dist():
    if dist.is_initialized():
        return
    cuda = torch.cuda.is_available()
    if "RANK" in os.environ:
        if cuda:
            local = int(os.environ.get("LOCAL_RANK", "0"))
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            dist.init_process_group("gloo")
    else:
        from .engine import init_single_process_group
        if cuda:
            torch.cuda.set_device(0)
        init_single_process_group()


def device_epoch_ms(fn, dev):
    """Run ``fn`` and return its duration in ms: CUDA events on GPUs, perf_counter on CPU; MAX over ranks."""
    if dev.type == "cuda":
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        e1.synchronize()
        ms = e0.elapsed_time(e1)
    else:
        t0 = time.perf_counter()
        out = fn()
        ms = (time.perf_counter() - t0) * 1e3
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return out, float(t.item())


def check_status_all_ranks(dev, world):
    """Read the device status word (an expired bounded wait of a peer-memory kernel) and make every rank stop together:
    the code is all-reduced with MAX, so a rank whose own waits were fine does not train on against a peer that gave up."""
    from ..ops import native
    code = int(native.status(dev).item())
    if world > 1:
        t = torch.tensor([code], dtype=torch.int32, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        worst = int(t.item())
    else:
        worst = code
    if worst != 0:
        native.status(dev).zero_()
        raise RuntimeError(f"gt_b200: a peer-memory wait expired on some rank (code {worst}; this rank's code {code}): the step that "
                           "followed read incomplete buffers, so training stops before its results are used or saved")


def _auto_grid(args, world, n, e_graph, f_in, rank):
    """--grid_auto / --head_auto: the white-box model's choice for this world size."""
    from ..perf import grid_select as gs
    token = bool(getattr(args, "virtual_node", False))
    e_attn = gs.attention_edges(n, e_graph, args.exp_deg) + (2 * n if token else 0)
    graph = gs.Graph(n, e_attn, e_graph + n, f_in, name=args.graph_name or args.synthetic or "graph", token=token)
    model = gs.Model(args.hidden or 256, args.heads or 8, args.layers or 4, bf16=args.bf16, with_gcn=not args.no_gcn,
                     transport=getattr(args, "comm", "nccl"))
    if args.head_auto:
        best = gs.select_layout(world, graph, model)
    else:
        best = gs.select_grid(world, graph, model, n_sub=max(args.stream_sub, 1), streamed=args.stream_sub > 1)
    if rank == 0:
        tag = "head_auto" if args.head_auto else "grid_auto"
        alts = ", ".join(f"{'x'.join(map(str, c.grid))} {c.ms:.1f} ms/{c.gb:.1f} GB" for c in best.ranked[:5])
        print(f"[{tag}] world={world} N={n} E_attn={e_attn} -> grid {'x'.join(map(str, best.grid))} "
              f"(predicted {best.ms:.1f} ms/epoch, {best.gb:.1f} GB peak); candidates: {alts}", flush=True)
    return list(best.grid)


def nccl_tune(args):
    """``--nccl_tune``: raise NCCL's channel count for ring collectives (``NCCL_MIN_NCHANNELS=16``, ``NCCL_ALGO=Ring``, only where the
    environment does not set them) BEFORE the communicators are created.  ``auto`` does so only when the job spans several machines
    and the column group of the grid crosses them (its reduce-scatter then runs over the network, the case the reference tunes:
    ``gt3d/gt3d/train/train_dist.py:230-280``), and never with ``--sparse_comm`` (the setting slows the all-to-all-v); inside one
    NVSwitch domain NCCL's defaults are kept.  ``on`` forces it, ``off`` skips it.  Returns the line that rank 0 prints."""
    from ..perf.grid_select import placement
    if args.nccl_tune == "off":
        return None
    world = int(os.environ.get("WORLD_SIZE", "1"))
    gpn = max(1, int(os.environ.get("LOCAL_WORLD_SIZE", str(world))))
    dims = list(args.grid) + [1] * (3 - len(args.grid))
    k, m = placement(dims[0], dims[1], dims[2], gpn)["col"]
    want = args.nccl_tune == "on" or (world > gpn and m > 1 and not args.sparse_comm)
    if want:
        os.environ.setdefault("NCCL_MIN_NCHANNELS", "16")
        os.environ.setdefault("NCCL_ALGO", "Ring")
    setting = f"NCCL_MIN_NCHANNELS={os.environ.get('NCCL_MIN_NCHANNELS')} NCCL_ALGO={os.environ.get('NCCL_ALGO')}" if want else "NCCL defaults"
    return f"[nccl_tune] {max(1, world // gpn)} machine(s), column group layout {k}x{m} -> {setting}"


def main(argv=None):
    args = parse_with_config(build_parser(), argv)
    head_grid = validate(args)
    tune_line = nccl_tune(args) if not dist.is_initialized() else None
    init_dist()
    if tune_line and dist.get_rank() == 0:
        print(tune_line, flush=True)
    rank, world = dist.get_rank(), dist.get_world_size()
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    if cuda and not args.no_tf32_matmul:
        torch.backends.cuda.matmul.allow_tf32 = True
    dtype = torch.bfloat16 if (args.bf16 and cuda) else torch.float32
    backend = args.backend or ("cuda" if cuda else "torch")
    torch.manual_seed(args.seed)
    from ..ops import native
    from ..parallel.collectives import set_transport
    from ..parallel.grid import make_grid
    from ..parallel.layers import dist_accuracy, dist_cross_entropy, set_step
    from ..utils.timers import enable_timers, timers
    from .checkpoint import load_checkpoint, save_checkpoint
    from .engine import TrainEngine
    from . import workloads as W
    if args.timers:
        enable_timers(True)
    heap = None
    if args.comm == "p2p" and world > 1:
        if cuda:
            from ..parallel.symm import SymmetricHeap
            heap = SymmetricHeap(dev, args.heap_mb << 20)
        else:                                               # CPU ranks of one machine: the same heap logic over shared host memory
            from ..parallel.symm_host import HostSymmetricHeap
            heap = HostSymmetricHeap(args.heap_mb << 20, record=args.check_protocol)
        set_transport(heap)

    def mem(tag, model=None):
        if rank == 0 and cuda:
            s = (f"[mem] {tag:28s} allocated {torch.cuda.memory_allocated() / 2 ** 30:6.2f} GB  peak {torch.cuda.max_memory_allocated() / 2 ** 30:6.2f} GB"
                 f"  reserved {torch.cuda.memory_reserved() / 2 ** 30:6.2f} GB")
            if model is not None and hasattr(model, "structure_bytes"):
                s += f"  graph structures {model.structure_bytes() / 2 ** 30:5.2f} GB"
            print(s, flush=True)

    extra_fw = {}
    label_classes = None
    if args.data is None:
        name = args.synthetic or ("cpu_small" if args.model == "exphormer" else None)
        if args.grid_auto or args.head_auto:
            from ..data.synthetic import workload_graph
            probe = workload_graph(name or "cpu_small", seed=args.seed, scale_down=args.scale_down)
            args.grid = _auto_grid(args, world, probe["n"], int(probe["edge_index"].shape[1]), probe["x"].shape[1], rank)
            head_grid = len(args.grid) == 3
            args.fused = args.fused or not head_grid
        if args.auto_ckpt and not head_grid and not args.checkpoint:
            from ..data.synthetic import workload_graph
            from ..perf import grid_select as gs
            probe = workload_graph(name or "cpu_small", seed=args.seed, scale_down=args.scale_down)
            e_g = int(probe["edge_index"].shape[1])
            args.checkpoint = gs.auto_checkpoint(args.grid[0], args.grid[1], gs.Graph(probe["n"], gs.attention_edges(probe["n"], e_g, args.exp_deg),
                                                 e_g + probe["n"], probe["x"].shape[1]), gs.Model(args.hidden or 256, args.heads or 8, args.layers or 4))
            if rank == 0:
                print(f"[auto_ckpt] per-layer activation checkpointing {'ON' if args.checkpoint else 'off'}", flush=True)
        if args.model == "exphormer":
            layer = "ring" if args.ring else ("streamed" if args.stream_sub > 1 else ("pipelined" if args.pipeline_sub > 1 else
                                                                                      ("fused" if args.fused else "plain")))
            build = W.exphormer_workload_streamed if args.stream_gen else W.exphormer_workload
            wl = build(name, args.grid, dev, dtype, seed=args.seed, scale_down=args.scale_down, exp_deg=args.exp_deg,
                                      virtual_node=args.virtual_node, dropout=args.dropout, backend=backend, layer=layer, norm=args.norm,
                                      **(dict(token_dense=True) if args.token_dense else {}),
                                      stream_sub=max(args.stream_sub, args.pipeline_sub), comm_bf16=args.comm_bf16 or args.bf16, heap=heap,
                                      layers=args.layers, hidden=args.hidden, heads=args.heads, with_gcn=not args.no_gcn,
                                      with_attn=not args.no_attn, gather_proj=args.gather_proj, checkpoint=args.checkpoint,
                                      stream_overlap=args.stream_overlap, stream_compact=not args.no_stream_compact,
                                      sparse_comm=args.sparse_comm, sparse_transport="pull" if heap is not None else "a2a",
                                      sparse_threshold=(args.sparse_threshold if args.sparse_threshold_row is None
                                                        else (args.sparse_threshold_row, args.sparse_threshold)))
        else:
            wl = W.variant_workload(args.model, name, args.grid, dev, dtype, seed=args.seed, scale_down=args.scale_down,
                                    dropout=args.dropout, backend=backend, comm_bf16=args.comm_bf16 or args.bf16, khop=args.khop,
                                    label_input=args.label_input, layers=args.layers, hidden=args.hidden, heads=args.heads,
                                    max_degree=args.max_degree if args.max_degree != 64 or not args.khop else None,
                                    ffn_mult=args.ffn_mult, checkpoint=args.checkpoint)
            if args.model == "graphormer":
                extra_fw = dict(degree_loc=wl["degree"], out_degree_loc=wl.get("out_degree"))
            label_classes = wl["cfg"]["classes"]
        grid, model = wl["grid"], wl["model"]
        args.hidden, args.layers, args.heads = (args.hidden or wl["cfg"]["hidden"], args.layers or wl["cfg"]["layers"],
                                                args.heads or wl["cfg"]["heads"])
        x_loc, y_loc = wl["x"].to(dev), wl["y"].to(dev)
        masks = {k: v.to(dev) for k, v in wl["masks"].items()}
        n, n_train, e_total = wl["num_nodes"], wl["n_train"], wl["num_attn_edges"]
    else:
        from ..data.expander import block_expander_edges
        from ..data.loader import grid_n_pad, load_partition, read_meta
        from ..models.exphormer_dist import DistExphormer
        from ..models import gt_variants as gv
        meta = read_meta(args.data)
        n, n_feat, n_cls = meta["num_nodes"], meta["num_features"], meta["num_classes"]
        if (args.grid_auto or args.head_auto) and meta.get("num_edges"):
            args.grid = _auto_grid(args, world, n, meta["num_edges"], n_feat, rank)
            head_grid = len(args.grid) == 3
        n_pad = meta["n_pad"] if meta["layout"] == "native" else grid_n_pad(meta, world, 4096)
        grid = make_grid(args.grid, n, n_pad=n_pad, layout=args.grid_layout).to(dev)
        part = load_partition(args.data, grid, dev)
        x_loc, y_loc, masks = part["x"].to(dtype), part["y"], part["masks"]
        gcn_blk, gcn_w = part["edge_index"], part["weight"]
        cnt = torch.tensor([int(masks["train"].sum()), part["num_local_edges"]], device=dev)
        dist.all_reduce(cnt)
        n_train, e_total = int(cnt[0]), int(cnt[1]) // max(getattr(grid, "p_heads", 1), 1)
        hidden, heads, layers = args.hidden or 80, args.heads or 2, args.layers or 4
        args.hidden, args.heads, args.layers = hidden, heads, layers
        if args.model == "exphormer":
            exp_blk = block_expander_edges(grid, n, args.exp_deg, seed=args.seed, device=dev)
            a_blk = torch.cat([gcn_blk, exp_blk], dim=1)
            a_et = torch.cat([torch.zeros(gcn_blk.shape[1], dtype=torch.long, device=dev), torch.ones(exp_blk.shape[1], dtype=torch.long, device=dev)])
            model = DistExphormer(grid, gcn_blk, a_blk, a_et, n_feat, hidden, n_cls, layers, heads, dropout=args.dropout, gnn_dropout=args.dropout,
                                  backend=backend, gcn_weight=gcn_w, checkpoint=args.checkpoint, fused=args.fused, norm=args.norm,
                                  comm_dtype=torch.bfloat16 if args.comm_bf16 else None, rs_dtype=torch.bfloat16 if args.rs_bf16 else None,
                                  pipeline_sub=args.pipeline_sub, stream_sub=args.stream_sub, ring=args.ring, with_gcn=not args.no_gcn,
                                  with_attn=not args.no_attn, gather_proj=args.gather_proj, stream_overlap=args.stream_overlap,
                                  stream_compact=not args.no_stream_compact, kernel_dtype=torch.bfloat16 if (args.kernel_bf16 or args.bf16) else None,
                                  sparse_comm=args.sparse_comm, sparse_threshold=args.sparse_threshold,
                                  sparse_transport="pull" if heap is not None else "a2a", heap=heap).to(dev)
        else:
            a_blk, a_et = gcn_blk, gv.type_local_block(grid, gcn_blk)
            token_row = None
            if args.model == "graphormer":
                tok_ei, tok_et = gv.token_edges_local(grid, n, dev)
                a_blk, a_et = torch.cat([a_blk, tok_ei], dim=1), torch.cat([a_et, tok_et])
                token_row = gv.token_owned_row(grid, n)
                d_in, _ = gv.owned_degrees(grid, a_blk, a_et, dev)
                extra_fw = dict(degree_loc=d_in)
            model = gv.DistGTVariant(grid, a_blk, a_et, n_feat, hidden, n_cls, layers, heads, model=args.model, dropout=args.dropout,
                                     backend=backend, checkpoint=args.checkpoint, num_classes_label=n_cls if args.label_input else None,
                                     max_degree=args.max_degree, token_row=token_row, ffn_mult=args.ffn_mult).to(dev)
            label_classes = n_cls
    for p in model.parameters():
        dist.broadcast(p.data, src=0)
    if rank == 0:
        print(f"data: N={n} (padded {grid.n_pad}, chunk {grid.chunk}) grid={tuple(args.grid)} backend={backend} E={e_total} "
              f"n_train={n_train} dtype={str(dtype).split('.')[-1]} comm={args.comm}", flush=True)
        if heap is not None and len(set(heap.hosts)) > 1:
            kinds = [("row", grid.row_group), ("column", grid.col_group)] + ([("head", grid.head_group)] if getattr(grid, "p_heads", 1) > 1 else [])
            print("[comm] " + str(len(set(heap.hosts))) + " machines: " + ", ".join(
                f"{k} group on {'peer memory' if heap.group_is_local(g) else 'NCCL'}" for k, g in kinds)
                + f", gradient all-reduce on {'peer memory' if heap.group_is_local(None) else 'NCCL'}", flush=True)
        if hasattr(model, "compaction_stats"):
            tot, ne = model.compaction_stats()
            if tot > 0:                                      # streamed / pipelined layers: how hypersparse the sub-blocks are
                print(f"[compact] attention (row, sub-block) pairs with edges: {ne}/{tot} = {100 * ne / tot:.1f}% "
                      "(the rows the compact-accumulate kernels visit)", flush=True)
        if args.sparse_comm and getattr(model, "sparse_info", None):
            inf = model.sparse_info
            print(f"[sparse_comm] row share {inf['row_share']:.3f} -> {'SPARSE' if inf['use_row'] else 'dense'}; "
                  f"col share {inf['col_share']:.3f} -> {'SPARSE' if inf['use_col'] else 'dense'}", flush=True)
    mem("after model build", model)
    use_graph = args.cuda_graph and cuda and not (args.label_input or args.profile or args.coll_stats or args.saved_census)
    eng = TrainEngine(model, lr=args.lr, weight_decay=args.weight_decay, total_steps=args.epochs, warmup=args.warmup,
                      use_graph=use_graph, heap=heap)
    start_epoch = 0
    if args.resume:
        start_epoch, _ = load_checkpoint(args.resume, model, eng)
        if rank == 0:
            print(f"[resume] {args.resume}: continuing at epoch {start_epoch}", flush=True)
    cstats = None
    if args.coll_stats:
        from ..utils.collstats import CollectiveStats
        cstats = CollectiveStats()

    def forward(train):
        if args.model == "exphormer":
            return model(x_loc), masks["train"], n_train
        label_feat, loss_mask, n_loss = None, masks["train"], n_train
        if args.label_input:
            vis = masks["train"] & (torch.rand(y_loc.shape[0], device=dev) < args.label_rate) if train else masks["train"]
            label_feat = torch.where(vis, y_loc, torch.full_like(y_loc, label_classes))
            if train:
                loss_mask = masks["train"] & ~vis
                c = torch.tensor([int(loss_mask.sum())], device=dev)
                dist.all_reduce(c)
                n_loss = max(int(c.item()), 1)
        return model(x_loc, label_feat, **extra_fw), loss_mask, n_loss

    def loss_fn():
        logits, loss_mask, n_loss = forward(True)
        return dist_cross_entropy(logits, y_loc, loss_mask, n_loss)

    if args.eval_only:
        if not args.resume:
            raise SystemExit("--eval_only evaluates a checkpoint: give --resume FILE")
        model.eval()
        if heap is not None:
            heap.begin_step()
        with torch.no_grad():
            (logits, _, _), ms = device_epoch_ms(lambda: forward(False), dev)
            acc = dist_accuracy(logits, y_loc, masks)
        if cuda:
            check_status_all_ranks(dev, world)
        if args.predict_out:
            lo, hi = grid.owned_range()
            mine = (int(lo), logits.argmax(dim=1).cpu())
            parts = [None] * world
            if world > 1:
                dist.all_gather_object(parts, mine)
            else:
                parts = [mine]
            if rank == 0:
                n_all = grid.num_nodes
                pred = torch.full((grid.n_pad,), -1, dtype=torch.long)
                for lo_r, p_r in parts:                              # head-axis replicas write the same values
                    pred[lo_r:lo_r + p_r.numel()] = p_r
                torch.save(dict(pred=pred[:n_all].clone(), num_nodes=n_all), args.predict_out)
        if rank == 0:
            print(f"EVAL checkpoint={args.resume} epoch={start_epoch} train={acc['train']:.4f} val={acc['valid']:.4f} test={acc['test']:.4f} "
                  f"forward_ms={ms:.2f} grid={'x'.join(map(str, args.grid))} world={world}", flush=True)
        return dict(eval=acc, epoch=start_epoch, forward_ms=ms)
    best = dict(val=-1.0, test=0.0, epoch=-1)
    host_ms = []                                             # host time to ENQUEUE a step (no synchronisation inside)

    def enqueue_step():
        t0 = time.perf_counter()
        out = eng.train_step(loss_fn)
        host_ms.append((time.perf_counter() - t0) * 1e3)
        return out
    epoch_ms = []
    hb = None
    if args.heartbeat > 0 and world > 1:
        from ..utils.health import Heartbeat
        hb = Heartbeat(timeout=args.heartbeat)
    if cuda:
        torch.cuda.reset_peak_memory_stats()
    for epoch in range(start_epoch, args.epochs):
        model.train()
        set_step(epoch)
        if epoch == start_epoch + 2:
            if cuda:
                torch.cuda.reset_peak_memory_stats()
            timers().reset()
        prof_ctx = contextlib.nullcontext()
        if args.profile and epoch == start_epoch + 2:
            from ..utils.profiling import kernel_profile
            prof_ctx = kernel_profile(rank, world)
        census_ctx = contextlib.nullcontext()
        if args.saved_census and epoch == start_epoch + 2:
            from ..utils.profiling import saved_tensor_census
            census_ctx = saved_tensor_census(grid, rank, hidden=args.hidden)
        if cstats is not None:
            cstats.begin_epoch()
        if hb is not None:                                    # before this epoch's launches: is every peer still there?
            hb.beat()
            hb.check(wait_for_first=60.0 if epoch == start_epoch else 0.0)
        with prof_ctx, census_ctx:
            if hb is not None:
                loss, ms = hb.guarded(device_epoch_ms, enqueue_step, dev)      # an exception here is announced to the peers
            else:
                loss, ms = device_epoch_ms(enqueue_step, dev)
        if cstats is not None:
            cstats.end_epoch(keep=epoch >= start_epoch + 2)
        epoch_ms.append(ms)
        if cuda:
            check_status_all_ranks(dev, world)            # device_epoch_ms has synchronised: the status word is final for this epoch
            if heap is not None and epoch == start_epoch:
                heap.check_symmetric()                        # once: every rank has made the same symmetric-heap allocations
        if epoch in (start_epoch, start_epoch + 2):
            mem(f"after step (epoch {epoch})", model)
        if epoch % args.eval_every == 0 or epoch == args.epochs - 1:
            model.eval()
            with torch.no_grad():
                acc = dist_accuracy(forward(False)[0], y_loc, masks)
            if acc["valid"] > best["val"]:
                best = dict(val=acc["valid"], test=acc["test"], epoch=epoch)
            loss_tot = loss.detach().clone().float()
            if world > 1:
                dist.all_reduce(loss_tot)
            if rank == 0 and args.metrics_jsonl:
                import json
                with open(args.metrics_jsonl, "a") as mf:
                    mf.write(json.dumps(dict(epoch=epoch, loss=float(loss_tot.item()), train=float(acc["train"]), val=float(acc["valid"]),
                                             test=float(acc["test"]), epoch_ms=float(ms), best_val=float(best["val"]),
                                             best_epoch=int(best["epoch"]), world=world, grid=list(args.grid))) + "\n")
            if rank == 0 and (epoch % 10 == 0 or epoch == args.epochs - 1):
                print(f"epoch {epoch:4d} loss {loss_tot.item():.4f} train {acc['train']:.4f} val {acc['valid']:.4f} test {acc['test']:.4f} "
                      f"| best val {best['val']:.4f} test {best['test']:.4f} @ {best['epoch']} | {sum(epoch_ms) / len(epoch_ms):.1f} ms/epoch train",
                      flush=True)
        if args.save and args.save_every and (epoch + 1) % args.save_every == 0:
            if cuda:
                torch.cuda.synchronize()
                check_status_all_ranks(dev, world)        # never write a checkpoint from a step whose peer wait expired
            save_checkpoint(args.save, model, eng, epoch + 1, dict(best=best))
    if cuda:
        torch.cuda.synchronize()
        check_status_all_ranks(dev, world)
    if args.save:
        save_checkpoint(args.save, model, eng, args.epochs, dict(best=best))
    if cstats is not None:
        cstats.report()
    if args.timers:
        timers().report(divide_by=max(len(epoch_ms) - 2, 1))
        # Host-side enqueue time of a step per rank (epochs 2+): close to the device time means the step is paced by the host (launch /
        # autograd bound; a captured step enqueues in a fraction of it); the spread over ranks is skew the collectives absorb
        # (the reference prints the same for its backward pass, gt3d/gt3d/train/train_dist.py:609-615,655-664).
        keep = host_ms[2:] if len(host_ms) > 2 else host_ms
        mine = torch.tensor([sum(keep) / max(len(keep), 1)], dtype=torch.float64, device=dev)
        every = [torch.zeros_like(mine) for _ in range(world)]
        if world > 1:
            dist.all_gather(every, mine)
        else:
            every = [mine]
        if rank == 0:
            vals = [float(v.item()) for v in every]
            print(f"[cpu] step enqueue ms per epoch: min {min(vals):.2f} max {max(vals):.2f} mean {sum(vals) / len(vals):.2f} | per rank: "
                  + " ".join(f"{v:.1f}" for v in vals), flush=True)
    steady = epoch_ms[2:] if len(epoch_ms) > 2 else epoch_ms
    peak = torch.tensor([torch.cuda.max_memory_allocated() / 2 ** 30 if cuda else 0.0], device=dev)
    if world > 1:
        dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(f"FINAL best_val={best['val']:.4f} test_at_best={best['test']:.4f} epoch={best['epoch']} epochs={args.epochs} "
              f"grid={'x'.join(map(str, args.grid))} world={world}", flush=True)
        print(f"STEADY model={args.model} grid={'x'.join(map(str, args.grid))} world={world} hidden={args.hidden} layers={args.layers} "
              f"ms_per_epoch={sum(steady) / max(len(steady), 1):.2f} peak_gb={peak.item():.2f} timing=device_max_over_ranks", flush=True)
    if heap is not None and heap.host:                       # unmap and delete the shared files once every rank is done with them
        native.check_status(dev)
        if args.check_protocol:
            rep = heap.check_recorded()                      # raises on an access that the recorded signals and waits do not order
            if rank == 0:
                print(f"[protocol] {rep.n_ops} recorded operations on {world} ranks: every access to shared memory is ordered", flush=True)
        dist.barrier()
        set_transport(None)
        heap.close()
    return dict(best=best, epoch_ms=epoch_ms)


if __name__ == "__main__":
    main()
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
