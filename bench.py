"""Headline benchmark: full-graph Exphormer training step (= one epoch) on the 169,343-node synthetic graph.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torch.distributed.run, one rank per GPU)
    python bench.py --impl reference ...                     the unmodified reference through its own API, same workload

Workload (BASELINE.json config 2): Exphormer, bf16 compute, 4 layers, hidden 256, 8 heads, FFN 2x, dropout 0.1;
Chung-Lu power-law graph (exponent 2.1) with 169,343 nodes and 1,166,243 directed edges, symmetrised, plus degree-4
expander edges and one virtual node; 128 features, 40 classes, 54/18/28 split; grids (row blocks x column blocks) 1x1 / 2x1 /
2x2 / 4x2.
A step is forward + loss + backward + gradient all-reduce + clip + AdamW on the whole graph.  The metric is
attention edges per second = (directed attention edges x layers) / step time, whole job; ``ms_per_step`` is the epoch time.
Synthetic data, random-init weights.  Timing: CUDA events on the launching stream, max over ranks, barrier +
synchronize on both sides; the step's working set (tens of ~87 MB activations) is far larger than the 126 MB L2, so no
explicit flush is needed between iterations.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = "exphormer_arxiv"
# (P_d, P_o) = (row blocks, column blocks).  The 8-GPU grid of the workload has the factors 2 and 4; this package orients it as
# its performance model selects (4 row blocks x 2 column blocks: measured 6.0 ms against 7.0 ms for 2 x 4, because the
# reduce-scattered payload row is twice as wide as the gathered input row).  The reference arm keeps the grids the benchmark
# configuration names for it (2 x 4 at 8 GPUs), which is also what it was measured with on this machine.
GRIDS = {1: (1, 1), 2: (2, 1), 4: (2, 2), 8: (4, 2)}
REFERENCE_GRIDS = {1: (1, 1), 2: (2, 1), 4: (2, 2), 8: (2, 4)}


class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx = float(parts[1])
            except ValueError:
                continue
            for nm, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from gt_b200.ops import native
    from gt_b200.parallel.layers import dist_cross_entropy
    from gt_b200.train.engine import TrainEngine, init_single_process_group
    from gt_b200.train.workloads import exphormer_workload

    if not torch.cuda.is_available():
        raise SystemExit("bench.py measures the sm_100a kernels and needs a CUDA device")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    else:
        init_single_process_group("nccl")
    rank = dist.get_rank()
    heap = None
    if world > 1 and args.comm == "p2p":
        # the peer-memory transport needs CUDA IPC between the ranks' devices; all ranks fall back to NCCL together if any fails
        from gt_b200.parallel.symm import SymmetricHeap
        ok = torch.ones(1, device=dev)
        try:
            heap = SymmetricHeap(dev, bytes_=args.heap_mb << 20)
        except Exception as exc:                             # noqa: BLE001
            ok.zero_()
            if rank == 0:
                print(f"[bench] symmetric heap unavailable ({exc}); using NCCL", file=sys.stderr, flush=True)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if not bool(ok.item()):
            heap, args.comm = None, "nccl"
    grid_shape = tuple(args.grid) if args.grid else GRIDS[world]
    wl = exphormer_workload(WORKLOAD, grid_shape, dev, torch.bfloat16, seed=0, heap=heap, scale_down=args.scale_down,
                            token_dense=args.token_dense)
    model, grid = wl["model"], wl["grid"]
    for p in model.parameters():
        dist.broadcast(p.data, src=0)
    eng = TrainEngine(model, lr=1e-3, weight_decay=1e-3, total_steps=args.steps * 2 + args.warmup * 2 + 8, warmup=2,
                      use_graph=not args.no_graph, graph_warmup=2, heap=heap)
    # static device inputs (the CUDA graph reads them); the end-to-end path refreshes them from pinned host memory
    x_host = wl["x"].pin_memory()
    y_host, m_host = wl["y"].pin_memory(), wl["masks"]["train"].pin_memory()
    x_dev, y_dev, m_dev = (torch.empty_like(t, device=dev) for t in (x_host, y_host, m_host))
    for d_, h_ in ((x_dev, x_host), (y_dev, y_host), (m_dev, m_host)):
        d_.copy_(h_)
    n_train = wl["n_train"]

    def loss_fn():
        return dist_cross_entropy(model(x_dev), y_dev, m_dev, n_train)

    model.train()
    launches = {}

    def step_device():
        return eng.train_step(loss_fn)

    def step_e2e():
        x_dev.copy_(x_host, non_blocking=True)
        y_dev.copy_(y_host, non_blocking=True)
        m_dev.copy_(m_host, non_blocking=True)
        return float(eng.train_step(loss_fn))             # device -> host read of the step's loss

    if args.e2e_prefetch:
        # opt-in: the same per-step transfers through the package's input pipeline (copy stream + staging buffers, loss read one
        # step later); the static tensors of the captured step are refreshed device-to-device
        from gt_b200.train.prefetch import AsyncScalar, InputPrefetcher
        pre = InputPrefetcher({"x": x_host, "y": y_host, "m": m_host}, dev)
        ring = AsyncScalar(dev)

        def step_e2e():                                   # noqa: F811
            st = pre.next()
            x_dev.copy_(st["x"], non_blocking=True)
            y_dev.copy_(st["y"], non_blocking=True)
            m_dev.copy_(st["m"], non_blocking=True)
            ring.push(eng.train_step(loss_fn))
            return ring.pop_previous()

    # warm-up (includes CUDA-graph capture); the launch census is taken on one of these steps
    for i in range(max(args.warmup, 3)):
        before = native.launch_count()
        step_device()
        launches[i] = native.launch_count() - before
    torch.cuda.synchronize()
    native.check_status(dev)
    per_step = max(launches.values())                     # calls recorded while the step ran eagerly / was captured

    def timed(fn, steps):
        sampler = ClockSampler(local)
        sampler.start()
        dist.barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.perf_counter()
        t0.record()
        last = None
        for _ in range(steps):
            last = fn()
        t1.record()
        torch.cuda.synchronize()
        wall = (time.perf_counter() - w0) * 1e3
        dist.barrier()
        ms = torch.tensor([t0.elapsed_time(t1), wall], device=dev, dtype=torch.float64)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms[0].item() / steps, ms[1].item() / steps, sampler.stop(), last

    ms_dev, _, clocks, loss = timed(step_device, args.steps)
    _, ms_e2e, clocks_e2e, loss_e2e = timed(step_e2e, args.steps)
    native.check_status(dev)
    if args.profile:
        # per-kernel device time of ONE more step of the same kind (a graph replay unless --no_graph), after the timed region
        from gt_b200.utils.profiling import kernel_profile
        dist.barrier()
        torch.cuda.synchronize()
        with open(f"{args.profile}.rank{rank}.txt", "w") as fh:
            with kernel_profile(0, world, top=45, file=fh):
                step_device()
    edges_layers = wl["num_attn_edges"] * wl["cfg"]["layers"]
    peak = torch.tensor([torch.cuda.max_memory_allocated() / 2 ** 30], device=dev)
    dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    if rank == 0:
        h2d = sum(t.numel() * t.element_size() for t in (x_host, y_host, m_host))
        out = {
            "metric": "full-graph train epoch: attention edges/s (E_attn x layers / epoch time), device-timed, max over ranks",
            "value": edges_layers / (ms_dev * 1e-3), "unit": "edges/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_dev, "epoch_s": ms_dev * 1e-3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded Chung-Lu graph, N(0,1) features, random-init weights)",
            "config": {"model": "Exphormer 4L h256 8 heads FFN2x dropout0.1 LayerNorm, fused 2D layer", "global_batch": wl["num_nodes"],
                       "seq_len": wl["num_nodes"], "nodes": wl["num_nodes"], "attn_edges": wl["num_attn_edges"],
                       "parallelism": "grid " + "x".join(map(str, grid_shape)), "grid": list(grid_shape),
                       "comm": args.comm if world > 1 else "none",
                       "cuda_graph": not args.no_graph, "scale_down": args.scale_down,
                       "global_token": "dense terms" if args.token_dense else "edges of the sparse blocks",
                       "grid_choice": ("default of this arm for %d GPUs: the benchmark's factorisation, row x column blocks oriented by the "
                                       "performance model (--grid runs any other; the reference arm keeps its own)" % world) if not args.grid
                       else "given with --grid",
                       "l2": "step working set (>2 GB of activations) exceeds the 126 MB L2; no explicit flush"},
            "clocks": clocks,
            "e2e": {"value": edges_layers / (ms_e2e * 1e-3), "unit": "edges/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4, "timing": "host wall clock around K steps (H2D of pinned inputs + step + loss read), max over ranks",
                    "clocks": clocks_e2e},
            "gpu_launches": per_step * args.steps, "gpu_launches_per_step": per_step,
            "launch_census": {k: v for k, v in sorted(native.LAUNCHES.items())},
            "loss": float(loss), "peak_gb": peak.item(), "impl": "gt_b200",
        }
        print(json.dumps(out), flush=True)
    finish(dist, [eng] + ([heap] if heap is not None else []))


def finish(dist, release=()):
    """Orderly exit: drop the captured CUDA graph (it keeps the communicator's captured collectives alive, and a communicator
    with live captured work can block in its teardown), close the symmetric heap, synchronise, meet at a barrier, destroy the
    process group in a helper thread and leave through the interpreter's normal shutdown.  Only if the teardown does not
    return within 20 s is the process ended without it (the result line is already printed)."""
    import gc
    import torch
    torch.cuda.synchronize()
    for obj in release:
        if hasattr(obj, "release_graph"):
            obj.release_graph()
    gc.collect()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    for obj in release:
        if hasattr(obj, "close"):
            obj.close()
    sys.stdout.flush()
    sys.stderr.flush()
    done = threading.Event()

    def teardown():
        try:
            dist.destroy_process_group()
        finally:
            done.set()

    th = threading.Thread(target=teardown, daemon=True)
    th.start()
    th.join(timeout=20.0)
    if not done.is_set():
        print("[bench] destroy_process_group did not return within 20 s; exiting without it", file=sys.stderr, flush=True)
        os._exit(0)
    sys.exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--e2e_prefetch", action="store_true",
                    help="end-to-end loop with the input pipeline of gt_b200.train.prefetch (default: copies and loss read on the step's stream)")
    ap.add_argument("--token_dense", action="store_true",
                    help="the global token as dense terms instead of 2 n edges (gt_b200/parallel/token_dense.py; same model and result; off by default)")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--comm", default="p2p", choices=["nccl", "p2p"], help="grid collectives: NCCL or the package's peer-memory kernels")
    ap.add_argument("--heap_mb", type=int, default=2048)
    ap.add_argument("--grid", type=int, nargs="+", default=None, metavar="P",
                    help="process grid P_d P_o (default: 1x1, 2x1, 2x2, 4x2 for 1, 2, 4, 8 GPUs); used by the grid-ranking measurements")
    ap.add_argument("--no_graph", action="store_true", help="run the step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--profile", default=None, metavar="PREFIX",
                    help="after timing, write the per-kernel device time of one more step to PREFIX.rank<r>.txt (not part of the timed region)")
    ap.add_argument("--scale_down", type=int, default=1, help="divide the graph size (profiling captures only; invalid as a bench value)")
    args = ap.parse_args()
    if args.impl == "reference":
        from baseline.reference_arm import run_reference
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
