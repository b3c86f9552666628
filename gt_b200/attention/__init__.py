"""Attention operator: edge-list specification, block structures and the two back-ends (``torch``: CPU / oracle,
``cuda``: hand-written sm_100a kernels)."""
from .csr import BlockCSR, SegmentPlan, build_csr, rows_of_edges  # noqa: F401
from .ref import masked_sparse_attention_ref  # noqa: F401


def get_backend(name: str):
    """Module implementing ``attn_fwd_partial / attn_bwd_partial / attn_bwd / normalize`` for ``name``."""
    if name == "torch":
        from . import backend_torch
        return backend_torch
    if name == "cuda":
        from . import backend_cuda
        return backend_cuda
    raise ValueError(f"unknown attention backend {name!r} (expected 'torch' or 'cuda')")
