"""Measured epoch times the performance model is checked against (never fitted to): one row per run of
``bench.py`` / ``train_dist`` on B200, device time, max over ranks.  Add rows as measurements come in."""

# ``skew``: time of the attention kernels on this graph's blocks over their time on random blocks of the same shape
# (gt_b200.bench.bench_attention_single_gpu --graph exphormer_arxiv vs --random 169344 4025926): a power-law graph with a
# global token has hub rows and columns that a uniformly random block does not.
ARXIV_CL = dict(name="exphormer_arxiv", n=169_344, e_graph=2_332_486, f_in=128, exp_deg=4, virtual_node=True, classes=40, skew=1.0)

MEASURED = [
    # graph, (hidden, heads, layers), grid, transport, measured ms per step (bench.py --grid, CUDA-graph step, device time, max over ranks)
    dict(graph=ARXIV_CL, model=(256, 8, 4), grid=(1, 1), transport="nccl", ms=19.66),
    dict(graph=ARXIV_CL, model=(256, 8, 4), grid=(2, 1), transport="p2p", ms=13.08),
    dict(graph=ARXIV_CL, model=(256, 8, 4), grid=(4, 1), transport="p2p", ms=8.42),
    dict(graph=ARXIV_CL, model=(256, 8, 4), grid=(2, 2), transport="p2p", ms=8.77),
    dict(graph=ARXIV_CL, model=(256, 8, 4), grid=(1, 4), transport="p2p", ms=11.36),
    dict(graph=ARXIV_CL, model=(256, 8, 4), grid=(4, 2), transport="p2p", ms=6.00),
    dict(graph=ARXIV_CL, model=(256, 8, 4), grid=(8, 1), transport="p2p", ms=6.47),
    dict(graph=ARXIV_CL, model=(256, 8, 4), grid=(2, 4), transport="p2p", ms=7.03),
    dict(graph=ARXIV_CL, model=(256, 8, 4), grid=(1, 8), transport="p2p", ms=10.47),
]

# The 1 x 1 row was re-measured at 18.62 ms after the backward passes began to hand the score gradients from the column pass to
# a K-only row pass; the multi-GPU rows and the attention constants of the model predate that change, so the table keeps 19.66.

# Latest measurement per grid where it is newer than the table above (used by gt_b200.bench.check_regression, not by the model).
LATEST_MS = {(1, 1): 18.62}

# Other benchmark configurations, measured with ``train_dist --synthetic`` (device-timed ms per epoch, max over ranks; peak GB of
# the busiest rank).  They are listed for reference: the time model is calibrated for the Exphormer layer and is not compared
# with them.
OTHER_CONFIGS = [
    dict(name="UniMP 3 x 128 x 4, label inputs, 2,449,029 nodes, 56.7 M attention edges", grid=(1, 1), ms=134.3, peak_gb=21.7),
    dict(name="UniMP 3 x 128 x 4, label inputs, 2,449,029 nodes, 56.7 M attention edges", grid=(2, 2, 2), ms=37.5, peak_gb=4.0),
    dict(name="Graphormer-node 6 x 512 x 16, sampled 2-hop mask, 1,000,000 nodes, 53.0 M attention edges, layer checkpointing", grid=(1, 1), ms=1122.7,
         peak_gb=26.2),
    dict(name="Graphormer-node 6 x 512 x 16, sampled 2-hop mask, 1,000,000 nodes, 53.0 M attention edges, layer checkpointing", grid=(4, 2), ms=424.7,
         peak_gb=6.3),
    dict(name="Exphormer 2 x 256 x 8 streamed (8 sub-blocks), R-MAT 4,194,304 nodes, 98.8 M attention edges", grid=(1, 1), ms=663.6, peak_gb=72.0),
    dict(name="Exphormer 2 x 256 x 8 streamed, R-MAT 4,194,304 nodes, 98.8 M attention edges", grid=(4, 2), ms=183.1, peak_gb=12.4),
]
