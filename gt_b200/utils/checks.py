"""Host-side validation of the structures the kernels index with.  The kernels trust their plans (no per-access bounds
checks on the hot path); these checks run once, when a block or plan is built from outside data, and in tests.  They are
the stand-in for a device sanitizer run: every index a kernel will form is checked against its extent here."""
import torch


class StructureError(ValueError):
    pass


def validate_block(blk, num_types=None):
    """CSR (and, when built, CSC) of a ``BlockCSR``: monotone row pointers that end at the edge count, source indices inside
    the column block, edge types inside the gate / bias table, type-sorted rows (the kernels cache the gate per type run)."""
    crow, col = blk.crow.long().cpu(), blk.col.long().cpu()
    if crow.numel() != blk.n_rows + 1 or int(crow[0]) != 0 or int(crow[-1]) != col.numel():
        raise StructureError(f"row pointers: {crow.numel()} entries for {blk.n_rows} rows, last {int(crow[-1]) if crow.numel() else None}, edges {col.numel()}")
    if crow.numel() > 1 and bool((crow[1:] < crow[:-1]).any()):
        raise StructureError("row pointers decrease")
    if col.numel() and (int(col.min()) < 0 or int(col.max()) >= blk.n_cols):
        bad = int(((col < 0) | (col >= blk.n_cols)).nonzero()[0])
        raise StructureError(f"source index {int(col[bad])} at edge {bad} outside the column block of {blk.n_cols} rows")
    if blk.etype is not None:
        et = blk.etype.long().cpu()
        if et.numel() != col.numel():
            raise StructureError("edge types and sources differ in length")
        if et.numel() and (int(et.min()) < 0 or (num_types is not None and int(et.max()) >= num_types)):
            raise StructureError(f"edge type outside [0, {num_types})")
    return True


def validate_segment_plan(plan, n_rows, n_edges):
    """Segments of a row / column plan: inside the edge range, rows inside the block, slots inside the scratch area."""
    for name in ("seg_row", "seg_beg", "seg_end", "seg_slot"):
        t = getattr(plan, name, None)
        if t is None:
            continue
        t = t.long().cpu()
        if name == "seg_row" and t.numel() and (int(t.min()) < 0 or int(t.max()) >= n_rows):
            raise StructureError("segment row outside the block")
        if name in ("seg_beg", "seg_end") and t.numel() and (int(t.min()) < 0 or int(t.max()) > n_edges):
            raise StructureError(f"{name} outside the edge range")
        if name == "seg_slot" and t.numel() and int(t.max()) >= max(plan.num_slots, 1) and int(t.max()) >= 0:
            raise StructureError("scratch slot outside the scratch area")
    return True


def validate_sparse_plan(plan):
    """``SparseRowPlan``: the rows asked from every peer exist there, counts are consistent."""
    n_blk = plan.g * plan.rows_per_rank
    need = plan.need_local.long().cpu() if hasattr(plan, "need_local") else None
    if need is not None and need.numel():
        if int(need.min()) < 0 or int(need.max()) >= n_blk:
            raise StructureError("needed row outside the gathered block")
        if bool((need[1:] <= need[:-1]).any()):
            raise StructureError("need set must be sorted and unique")
    if hasattr(plan, "send_idx") and plan.send_idx is not None and plan.send_idx.numel():
        s = plan.send_idx.long().cpu()
        if int(s.min()) < 0 or int(s.max()) >= plan.rows_per_rank:
            raise StructureError("a peer asks for a row outside this rank's chunk")
    return True
