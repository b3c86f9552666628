"""Expander edges for Exphormer.

``random_regular_expander_edges`` is the "Random-d" construction of the Exphormer paper: the union of ``degree``
random permutations, both directions, self loops removed (no spectral-gap selection loop: random regular graphs are
expanders with high probability).  Reference: ``gt3d/gt3d/data/expander.py:13``.

For partitioned graphs no rank may build the global edge list, so the permutations must be evaluable *pointwise*:
``KeyedPermutation`` is a keyed bijection on ``[0, n)`` (a balanced Feistel network over the next even power of two
with cycle walking), and ``block_expander_edges`` enumerates exactly the expander edges that fall into a rank's
(row block, column block) from the block's own id ranges, with no communication
(reference: ``FeistelPermutation`` / ``block_expander_edges``, ``expander.py:41-106``).
"""
import torch

_M32 = 0xFFFFFFFF


def _union_both_ways(ids: torch.Tensor, images) -> torch.Tensor:
    """Edge list of ``i -> image(i)`` and ``image(i) -> i`` for every image vector, fixed points dropped."""
    fwd = torch.cat([torch.stack([ids, img]) for img in images], dim=1)
    both = torch.cat([fwd, fwd.flip(0)], dim=1)
    return both[:, both[0] != both[1]]


def random_regular_expander_edges(num_nodes: int, degree: int, seed: int = 0, device="cpu") -> torch.Tensor:
    gen = torch.Generator().manual_seed(int(seed))
    images = [torch.randperm(num_nodes, generator=gen) for _ in range(degree)]
    return _union_both_ways(torch.arange(num_nodes), images).to(device)


def _round_fn(x: torch.Tensor, key: int) -> torch.Tensor:
    """32-bit avalanche hash of ``x`` under ``key`` (xorshift-multiply rounds, evaluated in int64)."""
    z = (x + key) & _M32
    z = ((z ^ (z >> 15)) * 0x2C1B3C6D) & _M32
    z = ((z ^ (z >> 12)) * 0x297A2D39) & _M32
    return (z ^ (z >> 15)) & _M32


class KeyedPermutation:
    """Deterministic bijection of ``[0, n)`` indexed by ``(seed, index)``, evaluated elementwise on int64 tensors."""

    def __init__(self, n: int, seed: int, index: int = 0, rounds: int = 4):
        self.n = int(n)
        width = max(2, (self.n - 1).bit_length())
        self.half = (width + 1) // 2
        self.mask = (1 << self.half) - 1
        g = torch.Generator().manual_seed((int(seed) << 20) ^ (int(index) * 7919 + 13))
        self.keys = torch.randint(0, 2 ** 31 - 1, (rounds,), generator=g).tolist()

    def _pass(self, x):
        hi, lo = x >> self.half, x & self.mask
        for key in self.keys:
            hi, lo = lo, hi ^ (_round_fn(lo, key) & self.mask)
        return (hi << self.half) | lo

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        y = self._pass(x.to(torch.int64))
        out_of_range = y >= self.n
        while bool(out_of_range.any()):                    # cycle walking: re-encrypt until the value lands in [0, n)
            y = torch.where(out_of_range, self._pass(y), y)
            out_of_range = y >= self.n
        return y


def keyed_expander_edges(num_nodes: int, degree: int, seed: int = 0, device="cpu") -> torch.Tensor:
    """Global edge list of the union of ``degree`` keyed permutations (both directions, no self loops)."""
    ids = torch.arange(num_nodes, device=device)
    return _union_both_ways(ids, [KeyedPermutation(num_nodes, seed, which)(ids) for which in range(degree)])


def block_expander_edges(grid, num_nodes: int, degree: int, seed: int = 0, device="cpu") -> torch.Tensor:
    """Edges of ``keyed_expander_edges(num_nodes, degree, seed)`` with destination in ``grid``'s row block and source
    in its column block, as LOCAL ``(col-local src, row-local dst)`` indices (same contract as ``grid.local_block``)."""
    c_lo, c_hi = grid.col_block_range()
    col_ids = torch.arange(c_lo, min(c_hi, num_nodes), device=device)
    row_ids = torch.cat([torch.arange(lo, min(hi, num_nodes), device=device) for lo, hi in grid.row_block_ranges()]) \
        if any(lo < num_nodes for lo, _ in grid.row_block_ranges()) else torch.zeros(0, dtype=torch.long, device=device)
    srcs, dsts = [], []
    for idx in range(degree):
        pi = KeyedPermutation(num_nodes, seed, idx)
        # forward edges (i -> pi(i)): the source must be one of my columns, the image one of my rows
        img = pi(col_ids)
        ok = (grid.owner_of(img)[0].to(device) == grid.r) & (img != col_ids)
        srcs.append(col_ids[ok]); dsts.append(img[ok])
        # reverse edges (pi(i) -> i): the destination i is one of my rows, the source pi(i) one of my columns
        img = pi(row_ids)
        ok = (img >= c_lo) & (img < c_hi) & (img != row_ids)
        srcs.append(img[ok]); dsts.append(row_ids[ok])
    src, dst = torch.cat(srcs), torch.cat(dsts)
    return torch.stack([grid.global_to_col_local(src), grid.global_to_row_local(dst)])
