"""Stand-in of ``torch_scatter.segment_csr`` on ``torch.segment_reduce`` (sum / max / mean / min over CSR segments of
dim 0; empty segments give 0 like torch_scatter)."""
import torch


def segment_csr(src, indptr, out=None, reduce="sum"):
    lengths = (indptr[1:] - indptr[:-1]).to(torch.int64)
    red = {"sum": "sum", "add": "sum", "max": "max", "min": "min", "mean": "mean"}[reduce]
    if src.shape[0] == 0:
        return src.new_zeros((lengths.numel(),) + tuple(src.shape[1:]))
    res = torch.segment_reduce(src.contiguous(), red, lengths=lengths, axis=0, unsafe=True)
    if red in ("max", "min"):
        res = torch.where(torch.isfinite(res), res, torch.zeros_like(res))
    return res
