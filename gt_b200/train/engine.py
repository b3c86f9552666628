"""Training engine: flat parameter / gradient storage, gradient all-reduce, global-norm clipping, AdamW, cosine LR with
warm-up, and whole-step CUDA-graph capture.

``TrainEngine(model, ...)`` re-points every parameter (and its ``.grad``) into two flat fp32 buffers, so that

* the data-parallel gradient reduction is ONE collective on the flat buffer (no concatenation / copy-back as in the
  reference's ``allreduce_grads``, ``gt3d/gt3d/dist/layers.py:309-324``); with a symmetric heap it is the package's own
  peer-read all-reduce kernel, otherwise NCCL / gloo;
* clipping + AdamW are two kernels over the flat space (``sq_norm`` + ``adamw_step``; the clip coefficient and the
  learning rate are read from a device tensor, so the kernels are identical every step);
* on CUDA the whole step (zero-grad, forward, loss, backward, reduction, optimizer, dropout-RNG advance) can be captured
  once in a CUDA graph and replayed: the full-graph workload is static, and at ~10 ms per step on a B200 the ~500 kernel
  launches of an eager step would otherwise cost as much as the kernels themselves.

On CPU tensors (gloo tests, the CPU baseline) the same engine drives ``torch.optim.AdamW`` semantics in plain torch ops.
"""
import atexit
import math
import os
import shutil
import tempfile

import torch
import torch.distributed as dist


def cosine_with_warmup(step, warmup, total):
    """LR factor: linear warm-up over ``warmup`` steps, then cosine decay to zero at ``total``."""
    if step < warmup:
        return (step + 1) / max(warmup, 1)
    prog = (step - warmup) / max(total - warmup, 1)
    return 0.5 * (1.0 + math.cos(math.pi * min(prog, 1.0)))


def init_single_process_group(backend=None):
    """A world of one rank (single-GPU runs use the same distributed model classes on a 1x1 grid)."""
    if dist.is_initialized():
        return
    backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    folder = tempfile.mkdtemp(prefix="gt_b200_pg_")
    atexit.register(shutil.rmtree, folder, True)             # the rendezvous file is of no use after the process
    dist.init_process_group(backend, init_method=f"file://{os.path.join(folder, 'store')}", rank=0, world_size=1)


class TrainEngine:
    HYPER_SLOTS = 32

    def __init__(self, model, lr=1e-3, weight_decay=1e-3, total_steps=100, warmup=5, max_grad_norm=1.0, betas=(0.9, 0.999),
                 eps=1e-8, group=None, use_graph=False, graph_warmup=3, heap=None):
        self.model = model
        self.params = [p for p in model.parameters() if p.requires_grad]
        self.lr, self.wd, self.total, self.warmup = lr, weight_decay, total_steps, warmup
        self.max_norm, self.betas, self.eps = max_grad_norm, betas, eps
        self.group, self.heap = group, heap
        if heap is not None:
            from ..parallel.collectives import set_transport
            set_transport(heap)
        self.step_count = 0
        dev = self.params[0].device
        self.device = dev
        self.cuda = dev.type == "cuda"
        # Flat layout.  A model may name groups of parameters that must lie next to each other (``flat_param_order``): the
        # fused layers read K | V | message | Q weights as ONE stacked matrix and write their gradients as one GEMM.  Every
        # parameter starts on a multiple of 8 elements, so the bf16 shadow of any matrix is a legal (16-byte aligned) TMA operand.
        order = list(model.flat_param_order()) if hasattr(model, "flat_param_order") else []
        seen = {id(p) for p in order}
        order += [p for p in self.params if id(p) not in seen]
        order = [p for p in order if p.requires_grad]
        self.params = order
        self.offsets, n = {}, 0
        for p in order:
            n = -(-n // 8) * 8
            self.offsets[id(p)] = n
            n += p.numel()
        n = -(-n // 8) * 8
        self.numel = n
        self.flat_p = torch.zeros(n, dtype=torch.float32, device=dev)
        # gradients live in the symmetric heap and are reduced by its kernels when every rank of the group is on this machine
        self.on_heap = heap is not None and (self.cuda or heap.host) and heap.group_is_local(group)
        self.flat_g = heap.empty(n, torch.float32, "grads") if self.on_heap else torch.zeros(n, dtype=torch.float32, device=dev)
        self.flat_m = torch.zeros_like(self.flat_p)
        self.flat_v = torch.zeros_like(self.flat_p)
        # bf16 shadow of the parameters, refreshed by the optimizer kernel: the GEMMs read it instead of casting every step
        shadow = self.cuda or (heap is not None and heap.host)   # host: the emulated transport, so that tests run the same operator path
        self.flat_p_bf16 = torch.zeros(n, dtype=torch.bfloat16, device=dev) if shadow else None
        for p in order:
            off, k = self.offsets[id(p)], p.numel()
            self.flat_p[off:off + k].copy_(p.data.reshape(-1).float())
            p.data = self.flat_p[off:off + k].view_as(p)
            p.grad = self.flat_g[off:off + k].view_as(p)
            if shadow:
                p._bf16 = self.flat_p_bf16[off:off + k].view_as(p)
            if self.cuda:
                p._direct_grad = True         # backward kernels may add into p.grad themselves and return no gradient to autograd
                p._site = 0x51700000 + off    # dropout site id: position in the flat space, not an address
        self.sync_shadow()
        if hasattr(model, "on_flat_layout"):
            model.on_flat_layout(self)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if self.cuda:
            self.hyper = torch.zeros(9, dtype=torch.float32, device=dev)
            # The host may run many steps ahead of the device (graph replays are enqueued without a sync), and an asynchronous
            # host-to-device copy reads pinned memory when it EXECUTES: each step therefore writes its own pinned slot, and a
            # slot is rewritten only after the event recorded behind its previous copy has completed.
            self._hyper_slots = torch.zeros(self.HYPER_SLOTS, 8, dtype=torch.float32).pin_memory()
            self._hyper_events = [None] * self.HYPER_SLOTS
            self.g_sum = heap.empty(self.numel, torch.float32, "grads_sum") if heap is not None else None
        elif self.on_heap:
            self.g_sum = heap.empty(self.numel, torch.float32, "grads_sum")
        self.use_graph = use_graph and self.cuda
        self.graph_warmup = graph_warmup
        self._graph = None
        self._static_loss = None
        self._warm_done = 0          # eager steps run by THIS engine (a resumed step_count must not skip the warm-up)

    # ---- pieces of a step --------------------------------------------------------------------------------------------
    def _set_hyper(self):
        t = self.step_count + 1
        lr = self.lr * cosine_with_warmup(self.step_count, self.warmup, self.total)
        self.cur_lr = lr
        if self.cuda:
            i = self._hyper_cursor = (getattr(self, "_hyper_cursor", -1) + 1) % self.HYPER_SLOTS
            if self._hyper_events[i] is not None:
                self._hyper_events[i].synchronize()
            h = self._hyper_slots[i]
            h[0], h[1], h[2], h[3], h[4] = lr, self.betas[0], self.betas[1], self.eps, self.wd
            h[5], h[6] = 1.0 - self.betas[0] ** t, 1.0 - self.betas[1] ** t
            h[7] = self.max_norm if self.max_norm else 0.0
            self.hyper[:8].copy_(h, non_blocking=True)
            ev = self._hyper_events[i] or torch.cuda.Event()
            ev.record()
            self._hyper_events[i] = ev

    def _reduce_grads(self):
        if self.world == 1:
            return self.flat_g
        if self.on_heap:
            if self.world <= 8 and os.environ.get("GT_GRAD_ALLREDUCE", "two_shot") == "two_shot":
                # one kernel per rank: reduce my slice from every member, store it to every member (2 n bytes per rank, no barrier)
                self.heap.all_reduce_two_shot("grads", "grads_sum", self.numel, group=self.group)
                return self.g_sum
            return self.heap.all_reduce(self.flat_g, self.g_sum, "grads", group=self.group)
        dist.all_reduce(self.flat_g, group=self.group)
        return self.flat_g

    def _optimizer(self, g):
        if self.cuda:
            from ..ops import native
            e = native.ext()
            self.hyper[8:9].zero_()
            e.sq_norm(g, self.hyper[8:9])
            e.adamw_step(self.flat_p, g, self.flat_m, self.flat_v, self.flat_p_bf16, self.hyper, None)
            native.advance_rng(self.device)
            return
        b1, b2 = self.betas
        t = self.step_count + 1
        gs = 1.0
        if self.max_norm:
            norm = g.norm().item()
            gs = min(1.0, self.max_norm / (norm + 1e-6))
        gg = g * gs
        self.flat_m.mul_(b1).add_(gg, alpha=1 - b1)
        self.flat_v.mul_(b2).addcmul_(gg, gg, value=1 - b2)
        self.flat_p.mul_(1 - self.cur_lr * self.wd)
        denom = (self.flat_v / (1 - b2 ** t)).sqrt_().add_(self.eps)
        self.flat_p.addcdiv_(self.flat_m / (1 - b1 ** t), denom, value=-self.cur_lr)
        self.sync_shadow()

    def _body(self, loss_fn):
        if self.heap is not None:
            self.heap.begin_step()
        self.flat_g.zero_()
        loss = loss_fn()
        loss.backward()
        g = self._reduce_grads()
        self._optimizer(g)
        return loss.detach()

    # ---- public ------------------------------------------------------------------------------------------------------
    def train_step(self, loss_fn):
        """Run one optimisation step; ``loss_fn()`` does the forward pass on (static) tensors and returns this rank's
        share of the loss.  Returns the detached loss tensor (no host synchronisation)."""
        self._set_hyper()
        if not self.use_graph:
            loss = self._body(loss_fn)
        elif self._graph is None and self._warm_done < self.graph_warmup:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                loss = self._body(loss_fn)
            torch.cuda.current_stream().wait_stream(side)
            self._warm_done += 1
        else:
            if self._graph is None:
                self._graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self._graph):
                    self._static_loss = self._body(loss_fn)
            self._graph.replay()
            loss = self._static_loss
        self.step_count += 1
        return loss

    def sync_shadow(self):
        """Refresh the bf16 shadow after the fp32 parameters were written by anything but the optimizer kernel (a loaded
        checkpoint, a broadcast)."""
        if self.flat_p_bf16 is not None:
            self.flat_p_bf16.copy_(self.flat_p)

    def span(self, params, what="bf16"):
        """``[sum rows, cols]`` view of consecutive 2-D parameters of equal width in the flat space: their bf16 shadow
        (``what='bf16'``), fp32 values (``'fp32'``) or gradient (``'grad'``).  Raises if they are not adjacent."""
        off0 = self.offsets[id(params[0])]
        off, cols = off0, params[0].shape[1]
        for p in params:
            if self.offsets[id(p)] != off or p.dim() != 2 or p.shape[1] != cols or (p.numel() % 8):
                raise ValueError("parameters are not adjacent in the flat layout")
            off += p.numel()
        buf = {"bf16": self.flat_p_bf16, "fp32": self.flat_p, "grad": self.flat_g}[what]
        return buf[off0:off].view(-1, cols)

    def release_graph(self):
        """Drop the captured step (and the collectives recorded in it); the next ``train_step`` runs eagerly and re-captures."""
        self._graph = None
        self._static_loss = None
        self._warm_done = 0

    def state_dict(self):
        return dict(step=self.step_count, m=self.flat_m[:self.numel].clone(), v=self.flat_v[:self.numel].clone())

    def load_state_dict(self, sd):
        self.step_count = int(sd["step"])
        self.flat_m[:self.numel].copy_(sd["m"])
        self.flat_v[:self.numel].copy_(sd["v"])
        self.sync_shadow()


def smoke_step(device):
    """One tiny forward + backward + optimizer step of the flagship model (bf16 Exphormer, fused layer, LayerNorm) on the
    native kernels; raises if a kernel reports a failure or the loss is not finite."""
    from ..data.expander import random_regular_expander_edges
    from ..data.synthetic import erdos_renyi, node_data, symmetrize, virtual_node_edges
    from ..models.exphormer_dist import DistExphormer, gcn_edges_with_self_loops
    from ..models.exphormer_ref import ExphormerRef
    from ..ops import native
    from ..parallel.grid import Grid2D
    from ..parallel.layers import dist_cross_entropy
    torch.cuda.set_device(device)
    init_single_process_group()
    n, f, hid, classes = 4096, 64, 128, 16
    ei = symmetrize(erdos_renyi(n, 6, seed=1), n)
    exp = random_regular_expander_edges(n, 3, seed=1)
    tok, _ = virtual_node_edges(n)
    x, y, masks = node_data(n + 1, f, classes, seed=2)
    grid = Grid2D(1, 1, n + 1).to(device)
    attn_ei, attn_et = ExphormerRef.build_attention_edges(ei, exp, tok)
    model = DistExphormer(grid, gcn_edges_with_self_loops(ei, n + 1), attn_ei, attn_et, f, hid, classes, 2, 4, dropout=0.1,
                          gnn_dropout=0.1, num_edge_types=3, backend="cuda", fused=True, norm="ln",
                          kernel_dtype=torch.bfloat16).to(device)
    eng = TrainEngine(model, total_steps=4, warmup=1)
    xb, yb, mb = x.to(device).to(torch.bfloat16), y.to(device), masks["train"].to(device)
    n_train = int(masks["train"].sum())
    for _ in range(2):
        loss = eng.train_step(lambda: dist_cross_entropy(model(xb), yb, mb, n_train))
    torch.cuda.synchronize()
    native.check_status(device)
    val = float(loss)
    if not math.isfinite(val):
        raise RuntimeError(f"smoke step produced a non-finite loss {val}")
    print(f"smoke ok: loss {val:.4f}")
