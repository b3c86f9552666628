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


BASE = ["--grid", "1", "1", "--synthetic", "exphormer_arxiv", "--scale_down", "32", "--fused", "--norm", "ln", "--bf16", "--virtual_node", "--layers", "2",
        "--hidden", "64", "--heads", "4", "--dropout", "0.0", "--warmup", "1"]


def test_trainer_command_line_on_a_gpu(tmp_path):
    """``train_dist`` end to end on one GPU with a captured step: save, evaluate the checkpoint only, write predictions and metrics."""
    import json
    from gt_b200.train.train_dist import main
    ck, pred, met = str(tmp_path / "ck.pt"), str(tmp_path / "pred.pt"), str(tmp_path / "m.jsonl")
    res = main(BASE + ["--epochs", "6", "--cuda_graph", "--save", ck, "--metrics_jsonl", met])
    assert len(res["epoch_ms"]) == 6 and all(t > 0 for t in res["epoch_ms"])
    rows = [json.loads(line) for line in open(met)]
    assert rows and rows[-1]["loss"] < rows[0]["loss"]
    ev = main(BASE + ["--epochs", "6", "--resume", ck, "--eval_only", "--predict_out", pred])
    blob = torch.load(pred)
    assert blob["pred"].numel() == blob["num_nodes"] and 0.0 <= ev["eval"]["valid"] <= 1.0 and ev["epoch"] == 6


def test_dense_token_and_streamed_generation_from_the_command_line():
    from gt_b200.train.train_dist import main
    a = main(BASE + ["--epochs", "4"])
    b = main(BASE + ["--epochs", "4", "--token_dense"])
    assert abs(a["best"]["val"] - b["best"]["val"]) < 0.05
    c = main(["--grid", "1", "1", "--synthetic", "exphormer_rmat26", "--scale_down", "16384", "--stream_gen", "--stream_sub", "2", "--fused", "--bf16",
              "--epochs", "3", "--hidden", "64", "--heads", "4", "--norm", "ln"])
    assert len(c["epoch_ms"]) == 3
