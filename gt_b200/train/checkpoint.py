"""Checkpoint save / resume in the state-dict format.

The model part of a checkpoint is exactly ``model.state_dict()`` with the reference's parameter names and fp32 tensors
(``edge_type_emb.weight, pre_lin.weight, layers.{i}.q.weight, ...``; see :mod:`gt_b200.models.exphormer_ref`), so a file
written here loads into ``ExphormerRef`` / ``UniMPRef`` / ``GraphormerNodeRef`` and vice versa.  Parameters are
replicated on every rank, so rank 0 writes the whole model.  Beyond the reference (which never writes a checkpoint,
``gt3d/gt3d/train/train_dist.py`` has no ``torch.save``) the file also carries what a resume needs: AdamW moments, the step
counter (LR schedule position), the epoch, the best-validation record and the RNG states.  Writes are atomic.
"""
import os

import torch
import torch.distributed as dist

FORMAT_VERSION = 1


def _flat_names(model, engine):
    """Parameter names in the order of the engine's flat buffers (the order of the saved AdamW moments)."""
    by_id = {id(p): n for n, p in model.named_parameters()}
    return [by_id[id(p)] for p in engine.params]


def save_checkpoint(path, model, engine=None, epoch=0, extra=None):
    """Rank 0 writes ``path`` atomically; all ranks synchronise afterwards."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    if rank == 0:
        sd = {k: v.detach().to("cpu", torch.float32 if v.is_floating_point() else v.dtype).clone() for k, v in model.state_dict().items()}
        blob = dict(format_version=FORMAT_VERSION, model=sd, epoch=int(epoch), extra=extra or {},
                    rng_cpu=torch.get_rng_state())
        if engine is not None:
            es = engine.state_dict()
            blob["optimizer"] = dict(step=es["step"], m=es["m"].cpu(), v=es["v"].cpu(),
                                     names=_flat_names(model, engine))
        if torch.cuda.is_available():
            from ..ops import native
            try:
                blob["rng_dropout"] = native.rng_state().cpu()
            except Exception:
                pass
        tmp = f"{path}.tmp{os.getpid()}"
        torch.save(blob, tmp)
        os.replace(tmp, path)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def load_checkpoint(path, model, engine=None, strict=True):
    """Load on every rank; returns ``(epoch, extra)``.  A bare state dict (e.g. saved from a reference model) is accepted."""
    blob = torch.load(path, map_location="cpu", weights_only=True)      # tensors, dicts, lists, numbers and strings only
    sd = blob["model"] if isinstance(blob, dict) and "model" in blob and "format_version" in blob else blob
    own = model.state_dict()
    missing = [k for k in own if k not in sd]
    unexpected = [k for k in sd if k not in own]
    if strict and (missing or unexpected):
        raise KeyError(f"checkpoint mismatch: missing {missing[:5]}, unexpected {unexpected[:5]}")
    bad = [f"{k}: checkpoint {tuple(sd[k].shape)} vs model {tuple(own[k].shape)}" for k in sd if k in own and sd[k].shape != own[k].shape]
    if bad:
        raise ValueError("checkpoint was written for a different configuration: " + "; ".join(bad[:4]))
    with torch.no_grad():
        for k, v in sd.items():
            if k in own:
                own[k].copy_(v.to(own[k].dtype))            # in place: parameters may be views of the engine's flat buffer
    if sd is blob:
        return 0, {}
    if engine is not None and "optimizer" in blob:
        opt = blob["optimizer"]
        names = _flat_names(model, engine)
        if "names" in opt and list(opt["names"]) != names:
            raise ValueError("checkpoint was written for a different configuration: the optimizer state covers other parameters "
                             f"(or another order) than this model: first difference near {next((a, b) for a, b in zip(list(opt['names']) + [None], names + [None]) if a != b)}")
        if opt["m"].numel() != engine.numel or opt["v"].numel() != engine.numel:
            raise ValueError(f"checkpoint was written for a different configuration: optimizer moments of {opt['m'].numel()} elements, "
                             f"model has {engine.numel} trainable elements")
        engine.load_state_dict(dict(step=blob["optimizer"]["step"], m=blob["optimizer"]["m"].to(engine.device),
                                    v=blob["optimizer"]["v"].to(engine.device)))
    if "rng_cpu" in blob:
        torch.set_rng_state(blob["rng_cpu"])
    if "rng_dropout" in blob and torch.cuda.is_available():
        from ..ops import native
        native.rng_state().copy_(blob["rng_dropout"])
    return int(blob.get("epoch", 0)), blob.get("extra", {})
