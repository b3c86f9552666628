"""Shared fixtures: seeded random graphs with adversarial structure (a hub row, empty rows)."""
import torch


def random_graph(n, avg_deg, seed=0, hub=True, empty=(3, 7), n_types=3):
    g = torch.Generator().manual_seed(seed)
    e = n * avg_deg
    src = torch.randint(0, n, (e,), generator=g)
    dst = torch.randint(0, n, (e,), generator=g)
    if hub:                                   # node 1 attends to everything, everything attends to node 2
        src = torch.cat([src, torch.arange(n), torch.full((n,), 2)])
        dst = torch.cat([dst, torch.full((n,), 1), torch.arange(n)])
    keep = torch.ones_like(src, dtype=torch.bool)
    for r in empty:
        keep &= dst != r
    src, dst = src[keep], dst[keep]
    key = torch.unique(dst * n + src)          # no duplicate edges
    dst, src = key // n, key % n
    et = torch.randint(0, n_types, (src.numel(),), generator=g)
    return torch.stack([src, dst]), et
