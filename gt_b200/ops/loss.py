"""Masked softmax cross-entropy on the native kernel: one pass computes this rank's share of the loss
(``sum_i mask_i nll_i / denom``) and the logits gradient, so backward is a scale of a stored tensor
(replaces ``F.cross_entropy`` of the reference's ``dist_cross_entropy``, ``gt3d/gt3d/dist/layers.py:290-298``)."""
import torch

from . import native


class _MaskedCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, mask, denom):
        logits = logits.contiguous()
        loss = torch.zeros(1, dtype=torch.float32, device=logits.device)
        dlogits = torch.empty_like(logits)
        native.ext().cross_entropy(logits, labels.contiguous(), mask.contiguous(), 1.0 / float(denom), loss, dlogits)
        ctx.save_for_backward(dlogits)
        return loss[0]

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        return dlogits * g.to(dlogits.dtype), None, None, None


def masked_cross_entropy(logits, labels, mask, denom):
    return _MaskedCE.apply(logits, labels, mask, denom)
