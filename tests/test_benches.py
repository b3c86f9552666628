"""The benchmark entry points run end to end on CPU ranks (tiny sizes): they are part of the product's tooling."""
import pytest

from dist_utils import run_dist


def _bench_worker(rank, world, argv):
    from gt_b200.bench.bench_dist_attention import main
    assert main(argv) > 0


@pytest.mark.parametrize("argv", [
    ["--grid", "2", "1", "--strategy", "gather", "--sparse_comm", "--coll_timers"],
    ["--grid", "1", "2", "--strategy", "gather_proj"],
    ["--grid", "2", "1", "--strategy", "ring_kv2"],
    ["--grid", "1", "1", "2", "--strategy", "head"],
], ids=["gather_sparse", "gather_proj", "ring_kv2", "head"])
def test_bench_dist_attention(argv):
    run_dist(_bench_worker, 2, argv + ["--graph", "cpu_small", "--scale_down", "4", "--hidden", "32", "--heads", "4", "--iters", "1"])


def _coll_worker(rank, world):
    from gt_b200.bench.bench_collectives import main
    res = main(["--rows", "512", "--width", "16", "--share", "0.3", "--iters", "1"])
    assert {"ag_nccl", "rs_nccl", "sparse_gather_a2a", "sparse_reduce_a2a", "ring_hop_2buf"} <= set(res)


def test_bench_collectives_on_gloo():
    run_dist(_coll_worker, 2)
