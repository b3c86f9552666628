"""GPU tests of host-side features that were written without access to a GPU.  They use torch operations and kernels that other
tests of this suite cover, and they are marked so that a first-run failure is reported (``xfail``) without ending a run that stops at
the first failure; a pass is reported as ``XPASS``.  The file sorts just before the allocation-free entry point's, which must stay last."""
import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.xfail(reason="not yet run on a GPU", strict=False)]


def test_dense_global_token_matches_token_edges_on_the_kernels():
    """One GPU, bf16, the fused operator: the model with the token as dense terms and the model with the token's edges in the sparse
    block, same weights, give the same logits and training losses within bf16 noise."""
    from gt_b200.ops import native
    from gt_b200.parallel.layers import dist_cross_entropy
    from gt_b200.train.engine import TrainEngine, init_single_process_group
    from gt_b200.train.workloads import exphormer_workload
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    init_single_process_group()
    outs, losses = {}, {}
    for dense in (False, True):
        native.seed_rng(77, dev)
        wl = exphormer_workload("exphormer_arxiv", (1, 1), dev, torch.bfloat16, scale_down=16, layers=2, hidden=128, heads=4, dropout=0.0,
                                token_dense=dense)
        model = wl["model"]
        assert (model.layers[0].token is not None) == dense
        x, y, m = wl["x"].to(dev), wl["y"].to(dev), wl["masks"]["train"].to(dev)
        model.eval()
        with torch.no_grad():
            outs[dense] = model(x).float().cpu()
        model.train()
        eng = TrainEngine(model, lr=1e-3, total_steps=8, warmup=1)
        losses[dense] = torch.stack([eng.train_step(lambda: dist_cross_entropy(model(x), y, m, wl["n_train"])).clone() for _ in range(4)]).float().cpu()
        torch.cuda.synchronize()
        native.check_status(dev)
    scale = outs[False].abs().max().item()
    assert (outs[True] - outs[False]).abs().max().item() < 3e-2 * scale
    assert (losses[True] - losses[False]).abs().max().item() < 3e-2
