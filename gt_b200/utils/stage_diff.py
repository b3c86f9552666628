"""Stage-by-stage comparison of a distributed model with the single-process reference model on the same weights and inputs: where
does a parity failure start?

Forward hooks record the output of the input stage and of every layer on both sides, the logits complete the list; the distributed side
holds the owned rows, which are compared with the same rows of the reference; the table gives the largest absolute difference
per stage over all ranks and the magnitude of the reference activations.  The first stage whose difference leaves the precision's
noise floor is where to look.  (The reference repository keeps ``tests/debug_*.py`` scripts that diff its model against the official
implementation stage by stage; this is the same aid between this package's distributed and reference models.)

    torchrun --nproc-per-node 4 -m gt_b200.utils.stage_diff --grid 2 2 --fused            # gloo ranks on CPU, fp64
    python -m gt_b200.utils.stage_diff --grid 1 1 --layers 3
"""
import argparse

import torch
import torch.distributed as dist


def stage_diff(model, ref, grid, x, ref_args):
    """``[(stage, max |dist - ref| over all ranks, max |ref|)]``; ``model(grid.take_owned(x))`` against ``ref(x, *ref_args)``."""
    got, want = {}, {}

    def keep(store, name):
        return lambda _m, _i, out: store.__setitem__(name, (out[0] if isinstance(out, tuple) else out).detach())

    hooks = []
    for side, store in ((model, got), (ref, want)):
        for i, layer in enumerate(side.layers):
            hooks.append(layer.register_forward_hook(keep(store, f"layer {i}")))
    orig_m, orig_r = model.pre_mp, ref.pre_mp
    model.pre_mp = lambda t: _tap(got, "input stage", orig_m(t))
    ref.pre_mp = lambda t: _tap(want, "input stage", orig_r(t))
    try:
        with torch.no_grad():
            out = model(grid.take_owned(x).to(next(model.parameters()).dtype if x.is_floating_point() else x.dtype))
            out_ref = ref(x, *ref_args)
    finally:
        for h in hooks:
            h.remove()
        model.pre_mp, ref.pre_mp = orig_m, orig_r
    got["logits"], want["logits"] = out.detach(), out_ref.detach()
    lo, hi = grid.owned_range()
    nv = max(min(hi, grid.num_nodes) - lo, 0)
    rows = []
    for name in ["input stage"] + [f"layer {i}" for i in range(len(model.layers))] + ["logits"]:
        a, b = got[name][:nv].double(), want[name][lo:lo + nv].double()
        err = torch.tensor([(a - b).abs().max().item() if nv else 0.0, want[name].abs().max().item()], dtype=torch.float64)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(err, op=dist.ReduceOp.MAX)
        rows.append((name, err[0].item(), err[1].item()))
    return rows


def _tap(store, name, value):
    store[name] = value.detach()
    return value


def main(argv=None):
    ap = argparse.ArgumentParser(description="per-stage difference between DistExphormer and ExphormerRef on a random graph")
    ap.add_argument("--grid", type=int, nargs="+", default=[1, 1])
    ap.add_argument("--nodes", type=int, default=200)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--hidden", type=int, default=32)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--fused", action="store_true")
    ap.add_argument("--norm", default="bn", choices=["bn", "ln", "rms"])
    ap.add_argument("--token", action="store_true", help="a global token (edges of type 2)")
    ap.add_argument("--token_dense", action="store_true", help="with --token --fused: the token as dense terms on the distributed side")
    ap.add_argument("--dtype", default="float64", choices=["float64", "float32"])
    args = ap.parse_args(argv)
    from ..data.expander import random_regular_expander_edges
    from ..data.synthetic import erdos_renyi, symmetrize, virtual_node_edges
    from ..models.exphormer_dist import DistExphormer
    from ..models.exphormer_ref import ExphormerRef, gcn_edges_with_self_loops
    from ..parallel.grid import make_grid
    from ..parallel.layers import set_step
    from ..train.engine import init_single_process_group
    import os
    if "RANK" in os.environ and not dist.is_initialized():
        dist.init_process_group("gloo")
    init_single_process_group("gloo")
    dt = getattr(torch, args.dtype)
    n = args.nodes
    ei = symmetrize(erdos_renyi(n, 4, seed=1), n)
    exp = random_regular_expander_edges(n, 2, seed=1)
    tok = virtual_node_edges(n)[0] if args.token else None
    n_tot = n + (1 if args.token else 0)
    torch.manual_seed(0)
    x = torch.randn(n_tot, 16, dtype=dt)
    nt = 3 if args.token else 2
    ref = ExphormerRef(16, args.hidden, 7, args.layers, args.heads, dropout=0.0, gnn_dropout=0.0, num_edge_types=nt, norm=args.norm).to(dt)
    world = dist.get_world_size()
    grid = make_grid(tuple(args.grid), n_tot, n_pad=-(-n_tot // (8 * world)) * 8 * world)
    dense = args.token and args.token_dense
    a_ei, a_et = ExphormerRef.build_attention_edges(ei, exp, None if dense else tok)
    a_blk, a_bt = grid.local_block(a_ei, a_et)
    g_blk, _ = grid.local_block(gcn_edges_with_self_loops(ei, n_tot))
    model = DistExphormer(grid, g_blk, a_blk, a_bt, 16, args.hidden, 7, args.layers, args.heads, dropout=0.0, gnn_dropout=0.0, num_edge_types=nt,
                          backend="torch", fused=args.fused, norm=args.norm, token_node=n if dense else None).to(dt)
    model.load_ref_state_dict(ref.state_dict())
    set_step(0)
    ref.eval(); model.eval()
    rows = stage_diff(model, ref, grid, x, (ei, exp, tok))
    if dist.get_rank() == 0:
        print(f"{'stage':<14} {'max |difference|':>18} {'max |reference|':>18}")
        for name, err, mag in rows:
            print(f"{name:<14} {err:>18.3e} {mag:>18.3e}")
    return rows


if __name__ == "__main__":
    main()
