"""gt_b200: full-graph training of structure-masked sparse graph transformers on NVIDIA B200.

Sub-packages
------------
attention   edge-list specification, CSR/CSC structures, the CPU torch backend and the sm_100a CUDA backend
data        synthetic graph generators, expander edges, streaming 2D partitioner and loaders
parallel    2D / 3D process grids, autograd collectives, symmetric heap + fused P2P kernels, distributed layers
models      Exphormer / UniMP / Graphormer-node references and their distributed counterparts
ops         python wrappers of the native kernels (GEMM, LayerNorm, SpMM, AdamW, loss, elementwise)
train       the `train_dist` / `train_single_gpu` command lines, checkpoint save / resume
perf        white-box performance + memory model and the grid chooser
utils       CUDA-event timers, collective statistics, logging helpers
"""

__version__ = "0.1.0"
