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
