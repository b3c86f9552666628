"""Python face of the sm_100a extension (``gt_b200/_ext/gt_b200_native*.so``, built by :mod:`gt_b200.build_ext`).

``ext()`` imports the prebuilt module and raises when it is missing on a machine that has a GPU: no operation of
this file falls back to a library kernel silently.  The wrappers allocate outputs / scratch with torch's caching
allocator, hand raw tensors to the launchers and wire the kernels into autograd:

    linear          tcgen05 GEMM with fused bias / ReLU / dropout epilogue; backward = tcgen05 GEMMs (input gradient on a
                    transposed weight copy, weight gradient with the split-K MN-major kernel)
    layer_norm      fused dropout + bias + residual + LayerNorm, forward and backward
    spmm            CSR aggregation and its transpose
    gemm_nt / gemm_nn / gemm_tn   raw GEMMs for the explicit-backward layers

Dropout masks are never stored: kernels regenerate them from ``(seed, step offset, site id)`` held in a device tensor
(``rng_state``), which keeps a whole training step capturable in one CUDA graph (the step offset is advanced on the
device by ``advance_rng``).
"""
import itertools
import os

import torch

_EXT = [None]
_GEMM_IMPL = os.environ.get("GT_GEMM", "tcgen05")      # "tcgen05" (default) | "cublas" (debug / comparison only)


LAUNCHES = {}          # entry point -> number of calls (every call enqueues at least one kernel of this package)


class _CountingExt:
    """Thin proxy of the extension module that counts the calls per entry point (the launch census of bench.py)."""

    def __init__(self, mod):
        self._mod = mod
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._mod, name)

            def fn(*a, _raw=raw, _name=name, **kw):
                LAUNCHES[_name] = LAUNCHES.get(_name, 0) + 1
                return _raw(*a, **kw)
            self._cache[name] = fn
        return fn


def launch_count() -> int:
    """Kernel-launching calls made so far (host-side helpers such as heap management are not counted)."""
    skip = ("heap_", "tensor_from_ptr", "attn_shape_supported", "_blocks")
    return sum(v for k, v in LAUNCHES.items() if not any(s in k for s in skip))


def ext():
    """The native module; raises if it has not been built."""
    if _EXT[0] is None:
        from .. import build_ext
        mod = build_ext.load_prebuilt()
        if mod is None:
            raise RuntimeError("gt_b200 native extension is not built: run `python -m gt_b200.build_ext` "
                               "(or __graft_entry__.build()) before using CUDA tensors")
        _EXT[0] = _CountingExt(mod)
    return _EXT[0]


# ---- per-device state: status word of the bounded waits, dropout RNG state -------------------------------------------
_STATE = {}


def _state(device):
    if torch.device(device).type == "cpu":                  # host emulation of the peer-memory transport (parallel/symm_host.py)
        key, dev = "cpu", torch.device("cpu")
    else:
        key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
        dev = torch.device("cuda", key)
    st = _STATE.get(key)
    if st is None:
        st = dict(status=torch.zeros(1, dtype=torch.int32, device=dev),
                  rng=torch.tensor([0x5EED, 0], dtype=torch.int64, device=dev))
        _STATE[key] = st
    return st


def status(device=None):
    return _state(device if device is not None else torch.cuda.current_device())["status"]


def check_status(device=None):
    """Raise if a kernel recorded an expired bounded wait (synchronises the device)."""
    code = int(status(device).item())
    if code == 0 and hasattr(ext()._mod, "attn_status"):
        code = int(ext()._mod.attn_status())           # bounded copy waits of the attention kernels (device-global word)
    if code != 0:
        status(device).zero_()
        raise RuntimeError(f"gt_b200 kernel reported an expired wait (code {code}): "
                           "1-3 GEMM producer/MMA/epilogue, 4-6 TN GEMM, 7 attention row copy, 8-10 tile attention producer/MMA/softmax, >=100 peer flag of rank code-100")


def rng_state(device=None):
    return _state(device if device is not None else torch.cuda.current_device())["rng"]


def seed_rng(seed: int, device=None):
    st = rng_state(device)
    st.copy_(torch.tensor([int(seed), 0], dtype=torch.int64))


def advance_rng(device=None):
    """Next step's dropout masks (device-side increment: legal inside a CUDA graph)."""
    rng_state(device)[1:2].add_(1)


_SITE = itertools.count(1)


def new_site() -> int:
    """A process-wide unique id for one dropout site (one per module instance and use)."""
    return next(_SITE)


def site_of(param, salt=0):
    """Dropout site id of the module that owns ``param``: the parameter's position in the training engine's flat space when
    there is one (identical models then draw identical masks, whatever their addresses), else its address."""
    base = getattr(param, "_site", None)
    if base is None:
        base = param.data_ptr()
    return (int(base) ^ salt) & 0xFFFFFFFFFF


def _dt_ok(t):
    return t.dtype in (torch.bfloat16, torch.float32)


# ---- GEMMs ---------------------------------------------------------------------------------------------------------------
def _rowmajor(t):
    if t.stride(-1) != 1 or (t.stride(0) % 8) or (t.data_ptr() % 16):
        t = t.contiguous()
    return t


def _pad_k(a, b):
    k = a.shape[1]
    if k % 8 == 0:
        return a, b
    pad = 8 - k % 8
    return torch.nn.functional.pad(a, (0, pad)), torch.nn.functional.pad(b, (0, pad))


_ACT = {None: 0, "relu": 1, "gelu": 2}


def gemm_nt(a, b, bias=None, act=None, p=0.0, site=0, out_dtype=None, out=None, accumulate=False):
    """``epilogue(a @ b^T)``: ``a [M, K]``, ``b [N, K]`` (bf16 -> tcgen05; fp32 -> cuBLAS, a plain library GEMM kept for
    fp32 parity runs).  ``bias`` fp32 ``[N]``; ``act`` in None/'relu'/'gelu'; dropout ``p`` at site id ``site``."""
    if a.dtype != torch.bfloat16 or _GEMM_IMPL == "cublas":
        y = a @ b.to(a.dtype).t()
        if bias is not None:
            y = y + bias.to(y.dtype)
        if act is not None or p > 0:
            y2 = torch.empty_like(y)
            pad = (-y.shape[1]) % 8
            if pad:
                raise ValueError("epilogue width must be a multiple of 8")
            ext().bias_act_dropout(y.contiguous(), None, y2, _ACT[act], float(p), rng_state(a.device), int(site))
            y = y2
        if out is not None:
            out.copy_(out + y if accumulate else y)
            return out
        return y.to(out_dtype) if out_dtype is not None else y
    a, b = _pad_k(a, b.to(torch.bfloat16))
    a, b = _rowmajor(a), _rowmajor(b)
    m, n = a.shape[0], b.shape[0]
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype or torch.bfloat16, device=a.device)
    if m == 0:
        return out
    ext().gemm_nt(a, b, out, bias.float() if bias is not None and bias.dtype != torch.float32 else bias, _ACT[act], float(p),
                  rng_state(a.device) if p > 0 else None, int(site), bool(accumulate), status(a.device))
    return out


def gemm_nn(a, w):
    """``a @ w``: ``a [M, N]``, ``w [N, K]`` (input gradients).  The small weight is transposed so that both operands of
    the tensor-core kernel are K-major."""
    return gemm_nt(a, w.t().contiguous())


def gemm_tn(a, b, out=None, accumulate=False):
    """``a^T @ b`` in fp32: ``a [M, N]``, ``b [M, K]`` -> ``[N, K]`` (weight gradients; reduction over the rows)."""
    if a.dtype != torch.bfloat16 or _GEMM_IMPL == "cublas" or (a.shape[1] % 8) or (b.shape[1] % 8):
        y = (a.t() @ b.to(a.dtype)).float()
        if out is not None:
            out.copy_(out + y if accumulate else y)
            return out
        return y
    a, b = _rowmajor(a), _rowmajor(b.to(torch.bfloat16))
    if out is None:
        out = torch.empty(a.shape[1], b.shape[1], dtype=torch.float32, device=a.device)
        accumulate = False
    if a.shape[0] == 0:
        return out if accumulate else out.zero_()
    ext().gemm_tn(a, b, out, bool(accumulate), status(a.device))
    return out


def weight_bf16(weight, dtype=torch.bfloat16):
    """``weight`` in the compute dtype: the training engine's bf16 shadow when there is one (refreshed by the optimizer kernel,
    so no cast runs per step), else a cast."""
    sh = getattr(weight, "_bf16", None)
    if sh is not None and dtype == torch.bfloat16:
        return sh
    return weight.to(dtype)


def direct_grad(param):
    """The fp32 gradient buffer a backward kernel may add into itself (the engine's flat gradient space), or None."""
    if getattr(param, "_direct_grad", False) and param.grad is not None and param.grad.dtype == torch.float32 and param.grad.is_contiguous():
        return param.grad
    return None


class _Linear(torch.autograd.Function):
    """y = drop(act(x W^T + b)).  Saved: x, W (bf16 copy), and y (ReLU: mask and dropout are read off y) or the
    pre-activation (GELU)."""

    @staticmethod
    def forward(ctx, x, weight, bias, act, p, site):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        wb = weight_bf16(weight, x2.dtype)
        ctx.weight, ctx.bias_param = weight, bias
        if act == "gelu":
            pre = gemm_nt(x2, wb, bias)
            y = torch.empty_like(pre)
            ext().bias_act_dropout(pre, None, y, 2, float(p), rng_state(x.device) if p > 0 else None, int(site))
            ctx.save_for_backward(x2, wb, pre)
        else:
            y = gemm_nt(x2, wb, bias, act, p, site)
            ctx.save_for_backward(x2, wb, y if (act == "relu" or p > 0) else None)
        ctx.cfg = (act, float(p), int(site), bias is not None, weight.dtype, shp)
        return y.view(*shp[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        x2, wb, aux = ctx.saved_tensors
        act, p, site, has_bias, wdt, shp = ctx.cfg
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        e = ext()
        dbias = None
        n = dy2.shape[0]
        if act is not None or p > 0 or has_bias:
            # dz = dy * act' * dropmask, with the bias gradient (column sums) as per-block partials
            part = torch.empty(e.colsum_blocks(n), dy2.shape[1], dtype=torch.float32, device=dy2.device) if has_bias else None
            if dy2.shape[1] % 8 == 0 and dy2.dtype in (torch.bfloat16, torch.float32) and n > 0:
                dz = torch.empty_like(dy2)
                code = 1 if act == "relu" else (2 if act == "gelu" else 0)
                src = aux if code != 0 else None
                if code == 0 and p > 0:
                    # identity activation with dropout: the mask is regenerated from the site id
                    pass
                e.bias_act_dropout_bwd(dy2, src, None, dz, code, p if code != 2 else 0.0, rng_state(dy2.device) if p > 0 else None,
                                       site, part)
                if has_bias:
                    gb = direct_grad(ctx.bias_param)
                    if gb is not None:
                        e.reduce_partials(part, gb, True)          # straight into the flat gradient buffer
                    else:
                        dbias = torch.empty(dy2.shape[1], dtype=torch.float32, device=dy2.device)
                        e.reduce_partials(part, dbias, False)
            else:
                dz = dy2
                if has_bias:
                    dbias = dy2.float().sum(0)
        else:
            dz = dy2
        dx = gemm_nn(dz, wb) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            gw = direct_grad(ctx.weight)
            if gw is not None and dz.dtype == torch.bfloat16 and _GEMM_IMPL != "cublas" and dz.shape[1] % 8 == 0 and x2.shape[1] % 8 == 0:
                gemm_tn(dz, x2, out=gw, accumulate=True)              # dW lands in the flat gradient buffer: no autograd add
            else:
                dw = gemm_tn(dz, x2).to(wdt)
        return (dx.view(shp) if dx is not None else None), dw, dbias, None, None, None


def linear(x, weight, bias=None, activation=None, dropout=0.0):
    site = site_of(weight)
    return _Linear.apply(x, weight, bias, activation, float(dropout), site)


# ---- fused dropout + bias + residual + LayerNorm -----------------------------------------------------------------------------
class _LayerNorm(torch.autograd.Function):
    """out = LN(x + dropout(y + ybias)).  ``x`` / ``ybias`` may be None.  With ``l`` given, ``y`` is the fp32 unnormalised
    attention accumulator ``acc [n, H * d_h]`` and the kernel uses ``y = acc / (l[head] + eps_l)`` (the attention
    normalisation is fused into the LayerNorm pass, forward and backward).  Saved: y, x, l, the row statistics."""

    @staticmethod
    def forward(ctx, y, x, ybias, gamma, beta, eps, p, site, l, eps_l):
        y = y.contiguous()
        x = x.contiguous() if x is not None else None
        acc_mode = l is not None
        like = x if acc_mode else y
        out = torch.empty_like(like)
        stats = torch.empty(y.shape[0], 2, dtype=torch.float32, device=y.device)
        yb = ybias.float() if ybias is not None else None
        lc = l.contiguous() if acc_mode else None
        ext().layer_norm_fwd(like if acc_mode else y, x, yb, gamma.float(), beta.float(), out, stats, float(eps), float(p),
                             rng_state(y.device) if p > 0 else None, int(site), y if acc_mode else None, lc, float(eps_l))
        ctx.save_for_backward(y, x, yb, gamma, stats, lc)
        ctx.cfg = (float(p), int(site), ybias is not None, beta.dtype, float(eps_l))
        return out

    @staticmethod
    def backward(ctx, dout):
        y, x, yb, gamma, stats, l = ctx.saved_tensors
        p, site, has_yb, pdt, eps_l = ctx.cfg
        e = ext()
        dout = dout.contiguous()
        n, d = y.shape
        acc_mode = l is not None
        like = x if acc_mode else y
        nb = e.layer_norm_bwd_blocks(n)
        parts = torch.empty(nb, 3, d, dtype=torch.float32, device=y.device)      # the block partials of all three sums side by side
        dy = torch.empty_like(y)                                  # acc mode: this is dacc (fp32)
        dl = torch.empty_like(l) if acc_mode else None
        dx = torch.empty_like(x) if x is not None else None
        e.layer_norm_bwd(dout, like if acc_mode else y, x, yb, gamma.float(), stats, like if acc_mode else dy, dx, False, parts[:, 0], parts[:, 1],
                         parts[:, 2], p, rng_state(y.device) if p > 0 else None, site,
                         y if acc_mode else None, l, eps_l, dy if acc_mode else None, dl)
        red = torch.empty(3, d, dtype=torch.float32, device=y.device)
        e.reduce_partials(parts.view(nb, 3 * d), red.view(3 * d), False)                # one reduction for dgamma | dbeta | dybias
        return dy, dx, (red[2].to(pdt) if has_yb else None), red[0].to(gamma.dtype), red[1].to(pdt), None, None, None, dl, None


def layer_norm(y, x, ybias, gamma, beta, eps, p, l=None, eps_l=1e-6):
    """``LayerNorm(x + dropout(y + ybias))`` over the last dimension of ``[n, d]`` tensors (d % 8 == 0, d <= 1024).
    ``l [n, H]``: ``y`` is an fp32 attention accumulator to be divided by ``l + eps_l`` per head first."""
    d = y.shape[-1]
    fused_ok = d % 8 == 0 and d <= 1024
    if l is not None:
        hd = d // l.shape[1]
        fused_ok = fused_ok and x is not None and y.dtype == torch.float32 and hd % 8 == 0 and ((hd // 8) & (hd // 8 - 1)) == 0
        if not fused_ok:
            y = (y.view(y.shape[0], l.shape[1], hd) / (l + eps_l).unsqueeze(-1)).reshape(y.shape).to(x.dtype if x is not None else y.dtype)
            l = None
            fused_ok = d % 8 == 0 and d <= 1024
    if not fused_ok:
        z = y + ybias.to(y.dtype) if ybias is not None else y
        z = torch.nn.functional.dropout(z, p, True) if p > 0 else z
        z = z + x if x is not None else z
        return torch.nn.functional.layer_norm(z, z.shape[-1:], gamma.to(z.dtype), beta.to(z.dtype), eps)
    site = site_of(gamma)
    return _LayerNorm.apply(y, x, ybias, gamma, beta, float(eps), float(p), site, l, float(eps_l))


class _GatedResidual(torch.autograd.Function):
    """UniMP combine in one kernel per direction (rows of up to 256 features); see ``csrc/rowops.cu``."""

    @staticmethod
    def forward(ctx, r, o, gate_weight, gate_bias, ln_weight, ln_bias, eps, p, site):
        d = r.shape[1]
        w = gate_weight.float().view(3, d)
        wa, wb = (w[0] + w[2]).contiguous(), (w[1] - w[2]).contiguous()
        r, o = r.contiguous(), o.to(r.dtype).contiguous()
        out = torch.empty_like(r)
        stats = torch.empty(r.shape[0], 3, dtype=torch.float32, device=r.device)
        ext().gated_res_fwd(r, o, wa, wb, gate_bias.float().reshape(1), ln_weight.float(), ln_bias.float(), out, stats, float(eps), float(p),
                            rng_state(r.device) if p > 0 else None, int(site))
        ctx.save_for_backward(r, o, wa, wb, ln_weight, ln_bias, stats)
        ctx.cfg = (float(p), int(site), gate_weight.dtype, gate_bias.dtype, gate_weight.shape)
        return out

    @staticmethod
    def backward(ctx, dout):
        r, o, wa, wb, gamma, beta, stats = ctx.saved_tensors
        p, site, wdt, bdt, wshape = ctx.cfg
        e = ext()
        d = r.shape[1]
        nb = e.premp_blocks(r.shape[0])
        part = torch.empty(nb, 4 * d + 8, dtype=torch.float32, device=r.device)
        dr, do_ = torch.empty_like(r), torch.empty_like(o)
        e.gated_res_bwd(r, o, dout.contiguous(), wa, wb, gamma.float(), beta.float(), stats, dr, do_, part, p,
                        rng_state(r.device) if p > 0 else None, site)
        red = torch.empty(4 * d + 8, dtype=torch.float32, device=r.device)
        e.reduce_partials(part, red, False)
        dwa, dwb = red[2 * d:3 * d], red[3 * d:4 * d]
        # wa = w0 + w2, wb = w1 - w2  ->  dw0 = dwa, dw1 = dwb, dw2 = dwa - dwb
        dw = torch.stack([dwa, dwb, dwa - dwb]).reshape(wshape).to(wdt)
        return dr, do_, dw, red[4 * d:4 * d + 1].to(bdt), red[:d].to(gamma.dtype), red[d:2 * d].to(beta.dtype), None, None, None


def gated_residual(r, o, gate_weight, gate_bias, ln_weight, ln_bias, eps, p):
    """UniMP combine ``drop(relu(LN(beta r + (1 - beta) o)))`` with ``beta = sigmoid(W_g [r | o | r - o] + b)``: one fused kernel per
    direction for rows of up to 256 features, otherwise two mat-vec products feeding the fused LayerNorm kernel."""
    d = r.shape[1]
    if d <= 256 and d % 8 == 0 and _dt_ok(r):
        site = site_of(gate_weight, 0x2545f491)
        return _GatedResidual.apply(r, o, gate_weight, gate_bias, ln_weight, ln_bias, eps, float(p), site)
    w = gate_weight.to(r.dtype).view(3, d)
    logit = r @ (w[0] + w[2]) + o @ (w[1] - w[2]) + gate_bias.to(r.dtype)
    beta = torch.sigmoid(logit).unsqueeze(-1)
    out = torch.relu(layer_norm(beta * r + (1.0 - beta) * o, None, None, ln_weight, ln_bias, eps, 0.0))
    return torch.nn.functional.dropout(out, p, True) if p > 0 else out


class _EmbedAdd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tab_a, idx_a, pad_a, tab_b, idx_b, pad_b):
        x = x.contiguous()
        out = torch.empty_like(x)
        ta = tab_a.float().contiguous()
        tb = tab_b.float().contiguous() if tab_b is not None else None
        ext().embed_add(x, ta, idx_a.contiguous(), int(pad_a), tb, idx_b.contiguous() if idx_b is not None else None, int(pad_b), out)
        ctx.save_for_backward(idx_a, idx_b)
        ctx.cfg = (tab_a.shape, tab_a.dtype, pad_a, tab_b.shape if tab_b is not None else None, tab_b.dtype if tab_b is not None else None, pad_b)
        return out

    @staticmethod
    def backward(ctx, dout):
        idx_a, idx_b = ctx.saved_tensors
        sa, da, pad_a, sb, db, pad_b = ctx.cfg
        dout = dout.contiguous()
        e = ext()
        dta = torch.zeros(sa, dtype=torch.float32, device=dout.device)
        e.embed_add_bwd(dout, idx_a.contiguous(), int(pad_a), dta)
        dtb = None
        if sb is not None:
            dtb = torch.zeros(sb, dtype=torch.float32, device=dout.device)
            e.embed_add_bwd(dout, idx_b.contiguous(), int(pad_b), dtb)
            dtb = dtb.to(db)
        return dout, dta.to(da), None, None, dtb, None, None


def embed_add(x, tab_a, idx_a, pad_a=-1, tab_b=None, idx_b=None, pad_b=-1):
    """``x + tab_a[idx_a] (+ tab_b[idx_b])`` row-wise in one pass; rows whose index is negative or equals ``pad`` get nothing."""
    return _EmbedAdd.apply(x, tab_a, idx_a, pad_a, tab_b, idx_b, pad_b)


SPMM_SEG = 256          # rows longer than this are cut into segments handled by separate warps


# ---- sparse ------------------------------------------------------------------------------------------------------------------
def spmm(blk, x, transpose=False, out=None):
    """``A @ x`` or ``A^T @ x`` for a BlockCSR with fp32 weights; ``out`` is accumulated into when given."""
    if x.shape[1] % 8 or x.shape[1] > 1024 or not _dt_ok(x):
        from .sparse import _spmm_torch
        if not transpose:
            return _spmm_torch(blk.rows().long(), blk.col.long(), blk.weight, x, blk.n_rows, out)
        ccol, rowidx, _, _, w_t = blk.csc()
        cols_of = torch.repeat_interleave(torch.arange(blk.n_cols, device=x.device), (ccol[1:] - ccol[:-1]).long())
        return _spmm_torch(cols_of, rowidx.long(), w_t, x, blk.n_cols, out)
    x = x.contiguous()
    if not transpose:
        ptr, idx, w, n_out, plan = blk.crow, blk.col, blk.weight, blk.n_rows, blk.row_plan(SPMM_SEG)
    else:
        ptr, idx, _, _, w = blk.csc()
        n_out, plan = blk.n_cols, blk.col_plan(SPMM_SEG)
    w = w if w.dtype == torch.float32 else w.float()
    acc = out is not None
    if out is None:
        out = torch.empty(n_out, x.shape[1], dtype=x.dtype, device=x.device)
    scratch = torch.empty(plan.num_slots, x.shape[1], dtype=torch.float32, device=x.device) if plan.num_slots else None
    ext().spmm(ptr, idx, w, x, out, acc, [plan.seg_row, plan.seg_beg, plan.seg_end, plan.seg_slot, plan.split_rows, plan.split_ptr],
               scratch, [], 0, 0, 0)
    return out


def segment_sum_rows(rows, perm, ptr, out):
    """``out[r] = sum_{k in [ptr[r], ptr[r+1])} rows[perm[k]]`` (deterministic)."""
    if rows.shape[1] % 8 or rows.shape[1] > 1024 or not _dt_ok(rows):
        seg = torch.repeat_interleave(torch.arange(out.shape[0], device=rows.device), (ptr[1:] - ptr[:-1]).long())
        return out.zero_().index_add_(0, seg, rows[perm.long()])
    ext().spmm(ptr, perm, None, rows.contiguous(), out, False, [], None, [], 0, 0, 0)
    return out


# ---- column packing (payloads of the row collectives) ---------------------------------------------------------------------
def pack_ok(parts):
    return all(t.is_cuda and t.dim() == 2 and t.dtype in (torch.float32, torch.bfloat16) and t.shape[1] % 8 == 0 for t in parts) \
        and 1 <= len(parts) <= 4


def pack_columns(parts, dtype):
    """``concat(parts, dim=1)`` converted to ``dtype`` in one pass (``parts``: ``[n, w_i]`` fp32 / bf16, ``w_i % 8 == 0``)."""
    parts = [_rowmajor(t) for t in parts]
    out = torch.empty(parts[0].shape[0], sum(t.shape[1] for t in parts), dtype=dtype, device=parts[0].device)
    if out.numel():
        ext().pack_cols(parts, out, True)
    return out


def unpack_columns(packed, widths, dtypes):
    """Inverse of :func:`pack_columns`: contiguous pieces ``[n, w_i]`` of the given dtypes."""
    packed = _rowmajor(packed)
    outs = [torch.empty(packed.shape[0], w, dtype=dt, device=packed.device) for w, dt in zip(widths, dtypes)]
    if packed.numel():
        ext().pack_cols(outs, packed, False)
    return outs


# ---- input stage: LayerNorm -> dropout -> ReLU -> L2 normalise in one kernel per direction ------------------------------------
class _PreMp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, gamma, beta, eps, p, site, l2norm):
        h = h.contiguous()
        out = torch.empty_like(h)
        stats = torch.empty(h.shape[0], 3, dtype=torch.float32, device=h.device)
        ext().premp_fwd(h, gamma.float(), beta.float(), out, stats, float(eps), float(p), rng_state(h.device) if p > 0 else None, int(site),
                        bool(l2norm))
        ctx.save_for_backward(h, gamma, beta, stats)
        ctx.cfg = (float(p), int(site), bool(l2norm))
        return out

    @staticmethod
    def backward(ctx, dout):
        h, gamma, beta, stats = ctx.saved_tensors
        p, site, l2norm = ctx.cfg
        e = ext()
        d = h.shape[1]
        nb = e.premp_blocks(h.shape[0])
        part = torch.empty(nb, 2 * d, dtype=torch.float32, device=h.device)
        dh = torch.empty_like(h)
        e.premp_bwd(h, dout.contiguous(), gamma.float(), beta.float(), stats, dh, part, p, rng_state(h.device) if p > 0 else None, site, l2norm)
        red = torch.empty(2 * d, dtype=torch.float32, device=h.device)
        e.reduce_partials(part, red, False)
        return dh, red[:d].to(gamma.dtype), red[d:].to(beta.dtype), None, None, None, None


def pre_mp(h, gamma, beta, eps, p, l2norm=True):
    """``l2normalize(relu(dropout(LayerNorm(h))))`` over the last dimension of ``[n, d]`` (d % 8 == 0, d <= 1024)."""
    site = site_of(gamma, 0x5bd1e995)
    return _PreMp.apply(h, gamma, beta, eps, float(p), site, bool(l2norm))
