"""Seeded synthetic graphs and node data of the shapes the benchmarks name.

Generators return a directed edge list ``[2, E]`` (row 0 = source, row 1 = destination) of int64 node ids; they run
on CPU or CUDA (``device=``) and are deterministic in ``seed`` for a given device type.

    erdos_renyi      G(n, m) with m = n * mean_degree directed edges
    chung_lu         expected-degree model with power-law weights (exponent gamma)
    rmat             recursive-matrix generator (a, b, c, d = 1 - a - b - c)
    symmetrize       add the reverse of every edge, drop duplicates
    add_self_loops   exactly one self loop per node (existing ones dropped first, PyG add_remaining_self_loops)
    virtual_node_edges   a global token connected both ways to every node
    khop_edges       the 2-hop mask A + A^2 with a shortest-path bucket per edge (0 self, 1 neighbour, 2 two hops)
    node_data        features / labels (uniform or Zipf) / train-val-test masks
"""
import math
from typing import Optional, Sequence

import torch


def _gen(seed: int, device) -> torch.Generator:
    return torch.Generator(device=device).manual_seed(int(seed))


def unique_edges(edge_index: torch.Tensor, n: int) -> torch.Tensor:
    """Drop duplicate (src, dst) pairs; result sorted by (dst, src)."""
    key = torch.unique(edge_index[1] * n + edge_index[0])
    return torch.stack([key % n, key // n])


def symmetrize(edge_index: torch.Tensor, n: int) -> torch.Tensor:
    both = torch.cat([edge_index, edge_index.flip(0)], dim=1)
    return unique_edges(both, n)


def add_self_loops(edge_index: torch.Tensor, n: int) -> torch.Tensor:
    keep = edge_index[0] != edge_index[1]
    loops = torch.arange(n, device=edge_index.device)
    return torch.cat([edge_index[:, keep], torch.stack([loops, loops])], dim=1)


def erdos_renyi(n: int, mean_degree: float, seed: int = 0, device="cpu") -> torch.Tensor:
    g = _gen(seed, device)
    m = int(round(n * mean_degree))
    ei = torch.randint(0, n, (2, m), generator=g, device=device)
    return ei[:, ei[0] != ei[1]]


def chung_lu(n: int, num_edges: int, gamma: float = 2.1, seed: int = 0, device="cpu") -> torch.Tensor:
    """``num_edges`` directed edges whose endpoints are drawn independently with probability proportional to the
    weights ``w_i = (i + i0)^(-1/(gamma-1))`` (a power-law expected-degree sequence with exponent ``gamma``).
    Sampling is by inverse CDF, so ``n`` is not limited by ``torch.multinomial``'s category cap."""
    g = _gen(seed, device)
    i0 = max(1.0, n ** (1.0 - 1.0 / (gamma - 1.0)) if gamma > 2 else 1.0)      # keeps the largest expected degree below ~sqrt(E)
    w = (torch.arange(n, dtype=torch.float64, device=device) + i0).pow(-1.0 / (gamma - 1.0))
    cdf = torch.cumsum(w, 0)
    cdf = cdf / cdf[-1]
    u = torch.rand(2, num_edges, dtype=torch.float64, generator=g, device=device)
    ei = torch.searchsorted(cdf, u).clamp_(max=n - 1)
    perm = torch.randperm(n, generator=g, device=device)                          # ids carry no degree order
    ei = perm[ei]
    return ei[:, ei[0] != ei[1]]


def rmat_chunks(scale: int, num_edges: int, a: float = 0.57, b: float = 0.19, c: float = 0.19, seed: int = 0, device="cpu",
                chunk: int = 1 << 26):
    """The edges of :func:`rmat` one chunk at a time (``[2, m]`` tensors, self loops removed): the same generator sequence, so
    concatenating the chunks gives exactly ``rmat(...)``.  For consumers that keep only a block of the graph."""
    g = _gen(seed, device)
    for e0 in range(0, num_edges, chunk):
        m = min(chunk, num_edges - e0)
        src = torch.zeros(m, dtype=torch.long, device=device)
        dst = torch.zeros(m, dtype=torch.long, device=device)
        for _ in range(scale):
            u = torch.rand(m, generator=g, device=device)
            right = ((u >= a) & (u < a + b)) | (u >= a + b + c)                 # quadrants b and d: column bit set
            down = u >= a + b                                                    # quadrants c and d: row bit set
            src = (src << 1) | right.long()
            dst = (dst << 1) | down.long()
        keep = src != dst
        yield torch.stack([src[keep], dst[keep]])


def rmat(scale: int, num_edges: int, a: float = 0.57, b: float = 0.19, c: float = 0.19, seed: int = 0, device="cpu",
         chunk: int = 1 << 26) -> torch.Tensor:
    """R-MAT graph on ``2**scale`` nodes: every bit of (src, dst) picks one of four quadrants with probabilities
    (a, b, c, 1-a-b-c).  Generated in chunks to bound the temporary memory."""
    parts = list(rmat_chunks(scale, num_edges, a, b, c, seed, device, chunk))
    return torch.cat(parts, dim=1) if parts else torch.zeros(2, 0, dtype=torch.long, device=device)


NODE_DATA_BLOCK = 1 << 16


def node_data_range(lo: int, hi: int, num_features: int, num_classes: int, split: Sequence[float] = (0.5, 0.25, 0.25), seed: int = 0,
                    device="cpu", dtype=torch.float32):
    """Node data of the nodes ``[lo, hi)`` of an arbitrarily large graph: ``(x ~ N(0,1), y uniform, masks)``.  Node ``i`` draws from
    the generator of its block ``i // 65536``, so any range, on any rank and any grid, yields the same values for the same node
    without generating the rest of the graph."""
    xs, ys, us = [], [], []
    for blk in range(lo // NODE_DATA_BLOCK, -(-hi // NODE_DATA_BLOCK) if hi > lo else lo // NODE_DATA_BLOCK):
        g = _gen(seed * 1_000_003 + blk + 1, device)
        x = torch.randn(NODE_DATA_BLOCK, num_features, generator=g, device=device, dtype=torch.float32)
        y = torch.randint(0, num_classes, (NODE_DATA_BLOCK,), generator=g, device=device)
        u = torch.rand(NODE_DATA_BLOCK, generator=g, device=device)
        a, b = max(lo, blk * NODE_DATA_BLOCK) - blk * NODE_DATA_BLOCK, min(hi, (blk + 1) * NODE_DATA_BLOCK) - blk * NODE_DATA_BLOCK
        xs.append(x[a:b]); ys.append(y[a:b]); us.append(u[a:b])
    if not xs:
        z = torch.zeros(0, device=device)
        return z.new_zeros(0, num_features).to(dtype), z.long(), {k: z.bool() for k in ("train", "valid", "test")}
    x, y, u = torch.cat(xs).to(dtype), torch.cat(ys), torch.cat(us)
    t0, t1 = split[0], split[0] + split[1]
    return x, y, {"train": u < t0, "valid": (u >= t0) & (u < t1), "test": u >= t1}


def virtual_node_edges(n: int, token: Optional[int] = None, device="cpu"):
    """Edges of a global token (default id ``n``) to and from every node ``0..n-1``: ``(edge_index, to_token_mask)``."""
    token = n if token is None else token
    nodes = torch.arange(n, device=device)
    tok = torch.full((n,), token, device=device, dtype=torch.long)
    ei = torch.cat([torch.stack([nodes, tok]), torch.stack([tok, nodes])], dim=1)
    to_tok = torch.cat([torch.ones(n, dtype=torch.bool, device=device), torch.zeros(n, dtype=torch.bool, device=device)])
    return ei, to_tok


def khop_edges(edge_index: torch.Tensor, n: int, max_two_hop: Optional[int] = None, seed: int = 0):
    """2-hop attention mask of a (symmetric) graph: self loops (bucket 0), neighbours (bucket 1) and nodes at
    shortest-path distance two (bucket 2).  ``max_two_hop`` caps the number of distance-2 sources kept per
    destination (a seeded random subset) so that hub neighbourhoods of scale-free graphs stay bounded; ``None`` keeps
    the exact ``A + A^2`` pattern.  Returns ``(edge_index, bucket)``."""
    dev = edge_index.device
    a = unique_edges(edge_index[:, edge_index[0] != edge_index[1]], n)
    key1 = a[1] * n + a[0]
    # two-hop candidates: join edges (j -> m) with (m -> i): sort by the middle node
    order_in = torch.argsort(a[1], stable=True)                                  # edges grouped by destination m
    m_sorted, j_sorted = a[1][order_in], a[0][order_in]
    in_ptr = torch.zeros(n + 1, dtype=torch.long, device=dev)
    torch.cumsum(torch.bincount(m_sorted, minlength=n), 0, out=in_ptr[1:])
    mid = a[0]                                                                   # for edge (m -> i): m is its source
    cnt = in_ptr[mid + 1] - in_ptr[mid]                                          # number of j with (j -> m)
    if max_two_hop is not None:
        g = _gen(seed, dev)
        # sample at most `max_two_hop` paths per destination by thinning every (m -> i) expansion proportionally
        deg_paths = torch.zeros(n, dtype=torch.float64, device=dev).index_add_(0, a[1], cnt.double())
        keep_p = (max_two_hop / deg_paths.clamp_min(1.0)).clamp_(max=1.0)[a[1]]
        take = torch.binomial(cnt.double(), keep_p, generator=g).long()
    else:
        take = cnt
    total = int(take.sum().item())
    eid = torch.repeat_interleave(torch.arange(a.shape[1], device=dev), take)
    first = torch.zeros(a.shape[1] + 1, dtype=torch.long, device=dev)
    torch.cumsum(take, 0, out=first[1:])
    k = torch.arange(total, device=dev) - first[eid]
    if max_two_hop is not None:
        g2 = _gen(seed + 1, dev)
        off = (torch.rand(total, generator=g2, device=dev, dtype=torch.float64) * cnt[eid].double()).long()
        off = torch.minimum(off, cnt[eid] - 1)
    else:
        off = k
    j = j_sorted[in_ptr[mid[eid]] + off]
    i = a[1][eid]
    key2 = torch.unique(i * n + j)
    key2 = key2[(key2 // n) != (key2 % n)]
    is_nb = torch.isin(key2, key1)
    key2 = key2[~is_nb]
    loops = torch.arange(n, device=dev)
    ei = torch.cat([torch.stack([loops, loops]), a, torch.stack([key2 % n, key2 // n])], dim=1)
    bucket = torch.cat([torch.zeros(n, dtype=torch.long, device=dev), torch.ones(a.shape[1], dtype=torch.long, device=dev),
                        torch.full((key2.numel(),), 2, dtype=torch.long, device=dev)])
    return ei, bucket


def node_data(n: int, num_features: int, num_classes: int, split: Sequence[float] = (0.5, 0.25, 0.25), labels: str = "uniform",
              zipf_s: float = 1.1, seed: int = 0, device="cpu", dtype=torch.float32):
    """``(x [n, F] ~ N(0,1), y [n] int64, masks {'train','valid','test'})``; labels uniform or Zipf(s)."""
    g = _gen(seed, device)
    x = torch.randn(n, num_features, generator=g, device=device, dtype=torch.float32).to(dtype)
    if labels == "uniform":
        y = torch.randint(0, num_classes, (n,), generator=g, device=device)
    elif labels == "zipf":
        w = torch.arange(1, num_classes + 1, dtype=torch.float64, device=device).pow(-zipf_s)
        cdf = torch.cumsum(w, 0) / w.sum()
        y = torch.searchsorted(cdf, torch.rand(n, dtype=torch.float64, generator=g, device=device)).clamp_(max=num_classes - 1)
    else:
        raise ValueError(labels)
    u = torch.rand(n, generator=g, device=device)
    t0, t1 = split[0], split[0] + split[1]
    masks = {"train": u < t0, "valid": (u >= t0) & (u < t1), "test": u >= t1}
    return x, y, masks


def degrees(edge_index: torch.Tensor, n: int):
    """(in_degree, out_degree) int64 [n]."""
    return torch.bincount(edge_index[1], minlength=n), torch.bincount(edge_index[0], minlength=n)


# ---------------------------------------------------------------------------------------------------------------
# The five benchmark workloads by name
# ---------------------------------------------------------------------------------------------------------------
WORKLOADS = {
    # name: (model, nodes, layers, hidden, heads, features, classes)
    "cpu_small": dict(model="exphormer", n=2_000, layers=2, hidden=64, heads=4, features=32, classes=10),
    "exphormer_arxiv": dict(model="exphormer", n=169_343, layers=4, hidden=256, heads=8, features=128, classes=40),
    "unimp_products": dict(model="unimp", n=2_449_029, layers=3, hidden=128, heads=4, features=100, classes=47),
    "graphormer_rmat": dict(model="graphormer", n=1_000_000, layers=6, hidden=512, heads=16, features=128, classes=64),
    "exphormer_rmat26": dict(model="exphormer", n=1 << 26, layers=2, hidden=256, heads=8, features=128, classes=172),
}


def workload_graph(name: str, seed: int = 0, device="cpu", scale_down: int = 1):
    """Base graph (symmetrised, no self loops / expander / token) and node data of a named workload.
    ``scale_down`` divides the node and edge counts (tests and smoke runs).  Returns a dict with ``edge_index, n, x, y,
    masks, num_classes`` and the workload's model hyper-parameters under ``cfg``."""
    cfg = dict(WORKLOADS[name])
    n = max(cfg["n"] // scale_down, 64)
    if name == "cpu_small":
        ei = symmetrize(erdos_renyi(n, 8, seed, device), n)
        split, lab = (0.5, 0.25, 0.25), "uniform"
    elif name == "exphormer_arxiv":
        ei = symmetrize(chung_lu(n, 1_166_243 // scale_down, 2.1, seed, device), n)
        split, lab = (0.54, 0.18, 0.28), "uniform"
    elif name == "unimp_products":
        ei = symmetrize(chung_lu(n, 61_859_140 // (2 * scale_down), 2.1, seed, device), n)
        split, lab = (0.08, 0.02, 0.90), "zipf"
    elif name == "graphormer_rmat":
        sc = max(int(math.log2(n)), 6)
        n = min(n, 1 << sc) if scale_down > 1 else cfg["n"]
        ei = rmat(sc, 16_000_000 // scale_down, seed=seed, device=device)
        ei = ei[:, (ei[0] < n) & (ei[1] < n)]
        ei = symmetrize(ei, n)
        split, lab = (0.5, 0.25, 0.25), "uniform"
    elif name == "exphormer_rmat26":
        sc = 26 - int(math.log2(scale_down)) if scale_down > 1 else 26
        n = 1 << sc
        ei = symmetrize(rmat(sc, (16 << sc) // 2, seed=seed, device=device), n)
        split, lab = (0.01, 0.01, 0.98), "uniform"
    else:
        raise KeyError(name)
    x, y, masks = node_data(n, cfg["features"], cfg["classes"], split, lab, seed=seed + 17, device=device)
    cfg["n"] = n
    return dict(edge_index=ei, n=n, x=x, y=y, masks=masks, num_classes=cfg["classes"], cfg=cfg)
