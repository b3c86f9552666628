"""The 1D strategies reproduce the single-process model (same seed, same graph): run with pytest, CPU ranks on gloo."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "tests"))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, strategy, expect):
    import dac26_sga
    res = dac26_sga.main(["--graph", "cpu_small", "--scale_down", "4", "--strategy", strategy, "--hidden", "32", "--heads", "4", "--layers", "2",
                          "--iters", "3", "--warmup", "0"])
    assert abs(res["first_loss"] - expect["first_loss"]) < 1e-4 * max(1.0, abs(expect["first_loss"])), (res, expect)
    assert abs(res["loss"] - expect["loss"]) < 1e-3 * max(1.0, abs(expect["loss"])), (res, expect)


@pytest.mark.parametrize("strategy", ["gp_ag", "gp_a2a"])
def test_strategies_match_single(strategy):
    import dac26_sga
    from dist_utils import run_dist
    single = dac26_sga.main(["--graph", "cpu_small", "--scale_down", "4", "--strategy", "single", "--hidden", "32", "--heads", "4", "--layers", "2",
                             "--iters", "3", "--warmup", "0"])
    run_dist(_worker, 2, strategy, single)


def test_micro_and_kernel_modes():
    import dac26_sga
    r = dac26_sga.main(["--graph", "cpu_small", "--scale_down", "4", "--micro", "--hidden", "32", "--heads", "4", "--iters", "1", "--warmup", "0"])
    assert {"mm_ms", "sddmm_ms", "spmm_ms"} <= set(r)
    r = dac26_sga.main(["--graph", "cpu_small", "--scale_down", "4", "--kernel", "--hidden", "32", "--heads", "4", "--iters", "1", "--warmup", "0"])
    assert r["fwd_bwd_ms"] > 0


def test_prepared_graph_files(tmp_path):
    import torch
    import dac26_sga
    import prepare_graphs
    paths = prepare_graphs.main(["--out", str(tmp_path), "--graphs", "proteins", "--scale_down", "400"])
    g = torch.load(paths[0], weights_only=True)
    assert g["num_nodes"] == 132_534 // 400 and g["edge_index"].shape[0] == 2 and int(g["edge_index"].max()) < g["num_nodes"]
    assert torch.equal(torch.unique(g["edge_index"][1] * g["num_nodes"] + g["edge_index"][0]).sort()[0],
                       torch.unique(g["edge_index"][0] * g["num_nodes"] + g["edge_index"][1]).sort()[0])      # symmetric
    torch.save(g["edge_index"], tmp_path / "raw.pt")
    again = prepare_graphs.main(["--out", str(tmp_path), "--name", "mine", "--edges", str(tmp_path / "raw.pt")])
    assert torch.equal(torch.load(again[0], weights_only=True)["edge_index"], g["edge_index"])
    r = dac26_sga.main(["--graph_file", paths[0], "--kernel", "--hidden", "32", "--heads", "4", "--iters", "1", "--warmup", "0"])
    assert r["nodes"] == g["num_nodes"] and r["fwd_bwd_ms"] > 0
