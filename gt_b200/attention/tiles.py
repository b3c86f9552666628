"""Density dispatch of a block's attention mask between two kernel families.

The gather kernels fetch one K and one V row per edge (1 KB per edge for 8 heads of 32 in bf16).  Where a 128 x 128 tile of
the mask holds more than a few percent of its entries, the tile's 128 K / V rows are cheaper to load once and multiply on the
tensor cores (``csrc/attn_tile.cu``).  Measured on B200 (16 heads of 32, biased softmax): 0.28-0.48 us per tile against
0.33 ns per gathered edge, so a tile pays from 6-10 % density.  :func:`tile_plan` splits a :class:`BlockCSR` into

* the tiles with at least ``min_edges`` edges, as a byte map per tile (edge type, 255 = no edge), grouped by row block, and
* the residual block (every other edge), which stays on the gather kernels.

The two contributions are partial softmax / clamp-exp states of the same rows and merge exactly.  The reference chooses
between its per-row and its tiled Triton kernels by edges per row (``gt3d/gt3d/attention/triton_kernel.py:530-578``); both of
those are gather kernels, and their regime is covered here by the persistent warp-per-segment kernels.  The split by tile
density is this package's second family.
"""
import os
from dataclasses import dataclass

import torch

from .csr import BlockCSR

TILE = 128
NO_EDGE = 255
MAX_TYPES = 15


def _env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


# GT_ATTN_TILE=0 turns the tensor-core family off; GT_ATTN_TILE_MIN = edges a tile must hold (default 10 % of 128 x 128: measured
# break-even against the gather kernels between 6 % with four dense tiles per row block and 10 % with one);
# GT_ATTN_TILE_SHARE = percent of the block's edges the dense tiles must cover before the second kernel is worth a launch
ENABLED = os.environ.get("GT_ATTN_TILE", "1") != "0"
MIN_EDGES = _env_int("GT_ATTN_TILE_MIN", 1638)
MIN_SHARE = _env_int("GT_ATTN_TILE_SHARE", 10) / 100.0
MAX_EDGES = _env_int("GT_ATTN_TILE_MAX_EDGES", 1 << 27)    # the split sorts one int64 key per edge: not attempted above this


@dataclass
class TilePlan:
    rb_ids: torch.Tensor        # int32 [n_rb]       row blocks that own at least one dense tile, ascending
    rb_ptr: torch.Tensor        # int32 [n_rb + 1]   range of tiles of every listed row block
    tile_cb: torch.Tensor       # int32 [n_tiles]    column block of every tile (ascending inside a row block)
    mask: torch.Tensor          # uint8 [n_tiles, 128, 128]  edge type of (row, column) inside the tile, 255 = no edge
    residual: BlockCSR          # the edges outside the dense tiles
    num_tiled_edges: int

    @property
    def num_tiles(self):
        return int(self.tile_cb.numel())


def build_tile_plan(blk: BlockCSR, min_edges=None, min_share=None):
    """Split ``blk`` into dense tiles and a residual block, or return ``None`` when no tile qualifies, the dense tiles cover less
    than ``min_share`` of the edges, an edge occurs twice inside a dense tile (a byte map cannot hold a multiplicity), or
    there are more than 15 edge types."""
    min_edges = MIN_EDGES if min_edges is None else int(min_edges)
    min_share = MIN_SHARE if min_share is None else float(min_share)
    e = blk.num_edges
    if e == 0 or e < min_edges or e > MAX_EDGES:
        return None
    if blk.etype is not None and e and int(blk.etype.max().item()) >= MAX_TYPES:
        return None
    dev = blk.device
    rows, cols = blk.rows().long(), blk.col.long()
    n_cb = (blk.n_cols + TILE - 1) // TILE
    key = (rows // TILE) * n_cb + cols // TILE
    uniq, inv, cnt = torch.unique(key, return_inverse=True, return_counts=True)       # ascending: by row block, then column block
    sel = cnt >= min_edges
    n_tiles = int(sel.sum().item())
    if n_tiles == 0:
        return None
    in_tile = sel[inv]
    n_in = int(in_tile.sum().item())
    if n_in < min_share * e:
        return None
    tile_of = torch.cumsum(sel.long(), 0) - 1
    flat = tile_of[inv][in_tile] * (TILE * TILE) + (rows[in_tile] % TILE) * TILE + cols[in_tile] % TILE
    if torch.unique(flat).numel() != flat.numel():
        return None
    mask = torch.full((n_tiles * TILE * TILE,), NO_EDGE, dtype=torch.uint8, device=dev)
    mask[flat] = blk.etype[in_tile].to(torch.uint8) if blk.etype is not None else torch.zeros(n_in, dtype=torch.uint8, device=dev)
    keys = uniq[sel]
    rb, cb = keys // n_cb, keys % n_cb
    rb_ids, rb_cnt = torch.unique_consecutive(rb, return_counts=True)
    rb_ptr = torch.zeros(rb_ids.numel() + 1, dtype=torch.long, device=dev)
    rb_ptr[1:] = torch.cumsum(rb_cnt, 0)
    keep = ~in_tile
    crow = torch.zeros(blk.n_rows + 1, dtype=torch.long, device=dev)
    crow[1:] = torch.cumsum(torch.bincount(rows[keep], minlength=blk.n_rows), 0)
    residual = BlockCSR.from_csr(crow, blk.col[keep], blk.etype[keep] if blk.etype is not None else None, n_cols=blk.n_cols)
    return TilePlan(rb_ids.to(torch.int32).contiguous(), rb_ptr.to(torch.int32).contiguous(), cb.to(torch.int32).contiguous(),
                    mask.view(n_tiles, TILE, TILE), residual, n_in)


def tile_plan(blk: BlockCSR):
    """The cached split of ``blk`` (``None`` when the block stays on the gather kernels alone)."""
    if not ENABLED:
        return None
    if "tile_plan" not in blk._cache:
        blk._cache["tile_plan"] = build_tile_plan(blk)
    return blk._cache["tile_plan"]


def tile_fwd_ref(q, k, v, plan: TilePlan, bias=None, *, score="dot", norm="softmax", clamp=(-5.0, 5.0), scale=None):
    """Dense-tile contribution as partial states ``(acc, l, m)`` with plain tensor operations (fp32): the oracle of the
    tensor-core kernel, tile by tile."""
    n, h, d = q.shape
    scale = d ** -0.5 if scale is None else float(scale)
    qf, kf, vf = q.float(), k.float(), v.float()
    acc = torch.zeros(n, h, d, dtype=torch.float32, device=q.device)
    l = torch.zeros(n, h, dtype=torch.float32, device=q.device)
    m = torch.full((n, h), float("-inf"), dtype=torch.float32, device=q.device) if norm == "softmax" else torch.zeros_like(l)
    rb_ptr = plan.rb_ptr.tolist()
    for i, rb in enumerate(plan.rb_ids.tolist()):
        r0, r1 = rb * TILE, min(n, rb * TILE + TILE)
        for t in range(rb_ptr[i], rb_ptr[i + 1]):
            c0 = int(plan.tile_cb[t]) * TILE
            c1 = min(k.shape[0], c0 + TILE)
            mk = plan.mask[t, :r1 - r0, :c1 - c0].long()
            has = mk != NO_EDGE
            s = torch.einsum("rhd,chd->hrc", qf[r0:r1], kf[c0:c1]) * scale
            if score == "biased" and bias is not None:
                s = s + bias.float()[mk.clamp(max=bias.shape[0] - 1)].permute(2, 0, 1)
            if norm == "softmax":
                s = s.masked_fill(~has, float("-inf"))
                mt = s.amax(-1).t()                                    # [rows, h]
                m_new = torch.maximum(m[r0:r1], mt)
                safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
                corr = torch.where(torch.isinf(m[r0:r1]), torch.zeros_like(m_new), torch.exp(m[r0:r1] - safe))
                p = torch.exp(s - safe.t()[:, :, None]).masked_fill(~has, 0.0)
                m[r0:r1] = m_new
            else:
                corr = torch.ones_like(l[r0:r1])
                p = torch.exp(s.clamp(clamp[0], clamp[1])).masked_fill(~has, 0.0)
            acc[r0:r1] = acc[r0:r1] * corr[:, :, None] + torch.einsum("hrc,chd->rhd", p, vf[c0:c1])
            l[r0:r1] = l[r0:r1] * corr + p.sum(-1).t()
    if norm == "softmax":
        m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    return acc, l, m
