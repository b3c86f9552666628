"""Stand-in of Plexus's row collectives: all-gather / reduce-scatter of 2-D tensors with an optional wire dtype."""
import torch
import torch.distributed as dist


def _all_gather_rows(x, group, wire_dtype=None, async_op=False):
    g = dist.get_world_size(group)
    src = x.to(wire_dtype) if wire_dtype is not None and wire_dtype != x.dtype else x
    src = src.contiguous()
    if g == 1:
        assert not async_op
        return src.to(x.dtype)
    out = src.new_empty((g * src.shape[0],) + tuple(src.shape[1:]))
    work = dist.all_gather_into_tensor(out, src, group=group, async_op=async_op)
    if async_op:
        return work, (lambda: out.to(x.dtype))
    return out.to(x.dtype)


def _reduce_scatter_rows(x, group, wire_dtype=None, async_op=False):
    g = dist.get_world_size(group)
    src = x.to(wire_dtype) if wire_dtype is not None and wire_dtype != x.dtype else x
    src = src.contiguous()
    if g == 1:
        return src.to(x.dtype)
    out = src.new_empty((src.shape[0] // g,) + tuple(src.shape[1:]))
    work = dist.reduce_scatter_tensor(out, src, group=group, async_op=async_op)
    if async_op:
        return work, (lambda: out.to(x.dtype))
    return out.to(x.dtype)
