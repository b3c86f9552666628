"""Measured epoch times the performance model is checked against (never fitted to): one row per run of
``bench.py`` / ``train_dist`` on B200, device time, max over ranks.  Add rows as measurements come in."""

ARXIV_CL = dict(name="exphormer_arxiv", n=169_344, e_graph=2_332_486, f_in=128, exp_deg=4, virtual_node=True, classes=40)

MEASURED = [
    # graph, (hidden, heads, layers), grid, transport, measured ms per step
    dict(graph=ARXIV_CL, model=(256, 8, 4), grid=(1, 1), transport="nccl", ms=43.5),
    dict(graph=ARXIV_CL, model=(256, 8, 4), grid=(2, 1), transport="nccl", ms=41.9),
    dict(graph=ARXIV_CL, model=(256, 8, 4), grid=(2, 1), transport="p2p", ms=41.6),
]
