"""Dense building blocks used by the models, with one implementation per device class.

On CUDA tensors every function runs the package's own sm_100a kernels (:mod:`gt_b200.ops.native`: tcgen05 GEMM with
fused bias / activation / dropout epilogues, fused dropout + residual + LayerNorm, ...) and raises if the extension is
not built.  On CPU tensors the same mathematics is expressed with PyTorch ops; that path is the oracle of the kernel
tests and carries the gloo multi-process tests.

    linear(x, w, b, activation, dropout)    y = drop(act(x w^T + b))
    dropout_add_norm(norm, y, x, bias, p)   norm(x + drop(y + bias))
    LayerNorm                               nn.LayerNorm whose CUDA forward / backward are the native kernels
    matmul_tn(a, b) = a^T b,  matmul_nn(a, b) = a b,  linear_nograd   (explicit-backward layers)
"""
import torch
import torch.nn as nn
import torch.nn.functional as F


def _native():
    from . import native
    return native


def _use_native(*tensors):
    return all(t is None or t.is_cuda for t in tensors) and any(t is not None for t in tensors) \
        and tensors[0].dtype in (torch.bfloat16, torch.float32)


def linear(x, weight, bias=None, activation=None, dropout=0.0, training=False):
    """``drop(act(x @ weight^T + bias))`` with ``activation`` in ``None | 'relu' | 'gelu'``.  ``weight`` is the fp32
    master parameter; the kernels read a bf16 copy when ``x`` is bf16."""
    if _use_native(x):
        return _native().linear(x, weight, bias, activation, dropout if training else 0.0)
    w = weight.to(x.dtype)
    y = F.linear(x, w, bias.to(x.dtype) if bias is not None else None)
    if activation == "relu":
        y = F.relu(y)
    elif activation == "gelu":
        y = F.gelu(y)
    elif activation is not None:
        raise ValueError(activation)
    return F.dropout(y, dropout, training) if dropout > 0 else y


@torch.no_grad()
def linear_nograd(x, weight):
    if _use_native(x):
        return _native().gemm_nt(x, weight.to(x.dtype))
    return x @ weight.to(x.dtype).t()


@torch.no_grad()
def matmul_tn(a, b):
    """``a^T @ b`` (weight gradients: ``a [M, N]``, ``b [M, K]`` -> ``[N, K]``), fp32 result for bf16 inputs."""
    if _use_native(a):
        return _native().gemm_tn(a, b)
    return a.t() @ b


@torch.no_grad()
def matmul_nn(a, w):
    """``a @ w`` (input gradients: ``a [M, N]``, ``w [N, K]``) in ``a``'s dtype."""
    if _use_native(a):
        return _native().gemm_nn(a, w.to(a.dtype))
    return a @ w.to(a.dtype)


class LayerNorm(nn.LayerNorm):
    """``nn.LayerNorm`` (same parameters / state-dict keys); CUDA inputs use the native row kernel."""

    def forward(self, x):
        if _use_native(x):
            return _native().layer_norm(x, None, None, self.weight, self.bias, self.eps, 0.0)
        return F.layer_norm(x, self.normalized_shape, self.weight.to(x.dtype), self.bias.to(x.dtype), self.eps)


def dropout_add_norm(norm, y, x, bias=None, p=0.0, training=False, l=None, eps_l=1e-6):
    """``norm(x + dropout(y + bias))``: the residual step of every branch.  Fused into one kernel for LayerNorm on CUDA.
    With ``l [n, H]`` given, ``y`` is the unnormalised attention accumulator ``[n, H * d_h]`` and is divided by
    ``l + eps_l`` per head first (inside the same kernel on CUDA)."""
    p = p if training else 0.0
    if isinstance(norm, LayerNorm) and _use_native(x):
        if l is not None:
            return _native().layer_norm(y.float(), x, bias, norm.weight, norm.bias, norm.eps, p, l.float(), eps_l)
        return _native().layer_norm(y.to(x.dtype), x, bias, norm.weight, norm.bias, norm.eps, p)
    if l is not None:
        h = l.shape[1]
        y = (y.reshape(y.shape[0], h, -1) / (l + eps_l).unsqueeze(-1)).reshape(y.shape[0], -1)
    y = y.to(x.dtype)
    if bias is not None:
        y = y + bias.to(x.dtype)
    if p > 0:
        y = F.dropout(y, p, True)
    return norm(x + y)


def gelu(x):
    return F.gelu(x)


def gated_residual(r, o, gate_weight, gate_bias, ln, p=0.0, training=False):
    """UniMP combine: ``beta = sigmoid(W_g [r | o | r - o] + b)``; ``drop(relu(LN(beta r + (1 - beta) o)))``.
    ``W_g [1, 3 dim]`` is split in three ``dim``-wide pieces so the concatenation is never materialised."""
    if _use_native(r) and isinstance(ln, LayerNorm):
        return _native().gated_residual(r, o, gate_weight, gate_bias, ln.weight, ln.bias, ln.eps, p if training else 0.0)
    d = r.shape[1]
    w = gate_weight.to(r.dtype).view(3, d)
    logit = r @ (w[0] + w[2]) + o @ (w[1] - w[2]) + gate_bias.to(r.dtype)
    beta = torch.sigmoid(logit).unsqueeze(-1)
    out = F.relu(ln(beta * r + (1.0 - beta) * o))
    return F.dropout(out, p, training) if p > 0 else out


class _SplitColumns(torch.autograd.Function):
    """Contiguous copies of consecutive column ranges of a 2-D tensor.  Backward is ONE concatenation of the pieces'
    gradients; autograd's own slice backward would allocate a zero matrix per piece and add them up."""

    @staticmethod
    def forward(ctx, x, *widths):
        ctx.widths, ctx.dtype = widths, x.dtype
        outs, c = [], 0
        for w in widths:
            outs.append(x[:, c:c + w].contiguous())
            c += w
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        ref = next(g for g in grads if g is not None)
        parts = [g if g is not None else ref.new_zeros(ref.shape[0], w) for g, w in zip(grads, ctx.widths)]
        return (torch.cat([p.to(ctx.dtype) for p in parts], dim=1),) + (None,) * len(ctx.widths)


def split_columns(x, widths):
    """``x [n, sum(widths)] -> tuple of contiguous [n, w]`` pieces."""
    if len(widths) == 1:
        return (x,)
    return _SplitColumns.apply(x, *widths)


def native_ok(x):
    """True when ``x`` takes the native row kernels (CUDA, bf16 / fp32, width a multiple of 8 up to 1024)."""
    return _use_native(x) and x.dim() == 2 and x.shape[1] % 8 == 0 and x.shape[1] <= 1024


def pre_mp(h, norm, p, l2norm=True):
    """Input stage ``l2normalize(relu(dropout(norm(h))))`` (dropout after the norm) as one native kernel per direction."""
    return _native().pre_mp(h, norm.weight, norm.bias, norm.eps, p, l2norm)


def embed_add(x, emb_a, idx_a, emb_b=None, idx_b=None):
    """``x + emb_a(idx_a) (+ emb_b(idx_b))`` for ``nn.Embedding`` modules (padding indices add nothing): one native pass on CUDA."""
    if native_ok(x):
        pad_a = emb_a.padding_idx if emb_a.padding_idx is not None else -1
        pad_b = emb_b.padding_idx if (emb_b is not None and emb_b.padding_idx is not None) else -1
        return _native().embed_add(x, emb_a.weight, idx_a, pad_a, emb_b.weight if emb_b is not None else None, idx_b, pad_b)
    out = x + emb_a(idx_a).to(x.dtype)
    if emb_b is not None:
        out = out + emb_b(idx_b).to(x.dtype)
    return out
