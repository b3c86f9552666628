"""The benchmark entry points run end to end on CPU ranks (tiny sizes): they are part of the product's tooling."""
import pytest

from dist_utils import run_dist


def _bench_worker(rank, world, argv):
    from gt_b200.bench.bench_dist_attention import main
    assert main(argv) > 0


@pytest.mark.parametrize("argv", [
    ["--grid", "2", "1", "--strategy", "gather", "--sparse_comm", "--coll_timers"],
    ["--grid", "1", "2", "--strategy", "gather_proj"],
    ["--grid", "2", "1", "--strategy", "ring_kv2"],
    ["--grid", "1", "1", "2", "--strategy", "head"],
], ids=["gather_sparse", "gather_proj", "ring_kv2", "head"])
def test_bench_dist_attention(argv):
    run_dist(_bench_worker, 2, argv + ["--graph", "cpu_small", "--scale_down", "4", "--hidden", "32", "--heads", "4", "--iters", "1"])


def _coll_worker(rank, world):
    from gt_b200.bench.bench_collectives import main
    res = main(["--rows", "512", "--width", "16", "--share", "0.3", "--iters", "1"])
    assert {"ag_nccl", "rs_nccl", "sparse_gather_a2a", "sparse_reduce_a2a", "ring_hop_2buf"} <= set(res)


def test_bench_collectives_on_gloo():
    run_dist(_coll_worker, 2)


# ---- single-process tools: need-set census, analytic tables, log / trace / capture post-processing -------------------------

def test_comm_sparsity_counts_match_the_poisson_model():
    import torch
    from gt_b200.bench import comm_sparsity as cs
    from gt_b200.bench.sparse_comm_model import need_share
    from gt_b200.data.synthetic import erdos_renyi, symmetrize
    n = 24000
    ei = symmetrize(erdos_renyi(n, 3, seed=1), n)
    deg = ei.shape[1] / n
    res = cs.survey(ei, n, [(4, 1), (2, 2)], orders=("native", "random"), exp_degree=2, token=False)
    for order in ("native", "random"):
        r41, r22 = res["orders"][order]
        assert abs(r41["col_need"]["mean"] - need_share(deg, 2, 4)) < 0.03
        assert abs(r22["col_need"]["mean"] - need_share(deg, 2, 2)) < 0.03
        assert abs(r22["row_need"]["mean"] - need_share(deg, 2, 2)) < 0.03
        assert r41["ring_need"]["mean"] >= r41["col_need"]["mean"]          # a hop carries the union over the other ranks
        assert 1.0 <= r41["balance"] < 1.3
    # a path graph in its native order references almost nothing across blocks; a random order does
    path = symmetrize(torch.stack([torch.arange(n - 1), torch.arange(1, n)]), n)
    res = cs.survey(path, n, [(4, 1)], orders=("native", "random", "bfs"), exp_degree=0, token=False)
    nat, rnd, bfs = (res["orders"][o][0]["col_need"]["mean"] for o in ("native", "random", "bfs"))
    assert nat < 0.01 and bfs < 0.01 and rnd > 0.3


def test_sparse_comm_model_table():
    from gt_b200.bench.sparse_comm_model import need_share, table
    assert need_share(10, 4, 1) == 1.0
    assert need_share(10, 0, 64) < need_share(10, 0, 8) < need_share(10, 0, 2) < 1.0
    rows = table([8, 64], [1, 4], degree=13.8, exp_degree=4)
    assert [r["grid"] for r in rows] == [[8, 1], [2, 4], [64, 1], [16, 4]]
    assert not rows[1]["use_col"] and rows[2]["use_col"]                    # 2 owners: dense; 64 owners: sparse pays
    assert not rows[0]["use_row"]                                          # a single column block has no Q-side gather


def test_regular_blocks_and_knee_fit():
    import torch
    from gt_b200.bench.kernel_theory import fit_knee, pass_bytes, regular_block
    for deg in (0, 1, 5):
        blk = regular_block(200, deg)
        crow = blk.crow.long()
        assert ((crow[1:] - crow[:-1]) == deg).all()
        assert (torch.bincount(blk.col.long(), minlength=200) == deg).all()
    fit = fit_knee([0, 1, 2, 4, 8, 16, 32, 64], [10, 10, 10, 11, 13, 20, 36, 68])
    assert abs(fit["ns_per_edge"] - 1.0) < 1e-9 and fit["floor_ns_per_row"] == 10 and abs(fit["knee_degree"] - 10) < 1e-9
    assert pass_bytes(100, 4, 256, 2)["bwd"] > pass_bytes(100, 4, 256, 2)["fwd"]


def test_ncu_report_joins_capture_and_order(tmp_path):
    from gt_b200.bench import kernel_ncu_report as rep
    head = '"ID","Kernel Name","gpu__time_duration.sum","dram__bytes_read.sum","dram__bytes_write.sum","launch__registers_per_thread"'
    units = '"","","us","Mbyte","Mbyte","register/thread"'
    rows = ['"0","void gt::attn_fwd_async_kernel<bf16>(AttnFwdArgs)","100","50","10","64"',
            '"1","attn_fwd_combine_sum_kernel(AttnFwdArgs)","5","1","1","32"',
            '"2","void gt::attn_bwd_row_kernel<bf16>(AttnBwdRowArgs)","200","90","20","106"',
            '"3","void gt::attn_bwd_col_kernel<bf16>(AttnBwdColArgs)","300","100","30","96"']
    cap = tmp_path / "cap.csv"
    cap.write_text("==PROF== banner\n" + "\n".join([head, units] + rows) + "\n")
    order = [dict(call="fwd", degree=16, model_bytes=31_000_000), dict(call="bwd", degree=16, model_bytes=120_000_000)]
    (tmp_path / "order.json").write_text(__import__("json").dumps(order))
    out = rep.main([str(cap), str(tmp_path / "order.json")])
    assert [r["kernels"] for r in out] == [2, 2]
    assert abs(out[0]["ms"] - 0.105) < 1e-9 and abs(out[0]["dram_bytes"] - 62e6) < 1 and abs(out[0]["dram_over_model"] - 2.0) < 1e-6
    assert out[1]["regs"] == 96 and abs(out[1]["dram_bytes"] - 240e6) < 1


def test_log_parsers_and_series(tmp_path):
    from gt_b200.bench import parse_logs, plot_figures
    log = tmp_path / "a.log"
    log.write_text(
        "data: N=100\n"
        "epoch    0 loss 3.8429 train 0.0258 val 0.0244 test 0.0258 | best val 0.0244 test 0.0258 @ 0 | 30.0 ms/epoch train\n"
        "epoch   10 loss 3.1000 train 0.2000 val 0.1900 test 0.1800 | best val 0.1900 test 0.1800 @ 10 | 20.0 ms/epoch train\n"
        "STEADY model=exphormer grid=1x1 world=1 hidden=256 layers=4 ms_per_epoch=26.50 peak_gb=4.44 timing=device_max_over_ranks\n"
        'ATTN {"nodes": 10, "fwd_ms": 0.9, "cfg": {"a": 1}}\n'
        'THEORY {"degree": 4, "fwd_ns_per_row": 1.5, "bwd_ns_per_row": 4.0}\n')
    log2 = tmp_path / "b.log"
    log2.write_text("STEADY model=exphormer grid=2x1 world=2 hidden=256 layers=4 ms_per_epoch=18.10 peak_gb=2.5 timing=device_max_over_ranks\n"
                    "STEADY model=exphormer grid=1x2 world=2 hidden=256 layers=4 ms_per_epoch=19.00 peak_gb=2.5 timing=device_max_over_ranks\n")
    cur = parse_logs.curves([str(log)])
    assert [r["epoch"] for r in cur] == [0, 10] and abs(cur[1]["train_seconds"] - 0.22) < 1e-9 and cur[1]["best_epoch"] == 10
    st = parse_logs.steady([str(log), str(log2)])
    assert st[0]["hidden"] == 256 and st[0]["ms_per_epoch"] == 26.5 and st[1]["grid"] == "2x1"
    lines = parse_logs.tagged_lines([str(log)], "ATTN")
    assert len(lines) == 1 and lines[0]["fwd_ms"] == 0.9 and lines[0]["cfg"] == '{"a": 1}'
    series = plot_figures.scaling_series(st)
    (key, pts), = series.items()
    assert key == ("exphormer", 256, 4) and pts == [(1, 26.5, "1x1"), (2, 18.1, "2x1")]
    eff = plot_figures.efficiency(pts)
    assert abs(eff[1][1] - 26.5 / (2 * 18.1)) < 1e-9
    assert plot_figures.sweep_series(parse_logs.tagged_lines([str(log)]))["bwd"] == [(4, 4.0)]
    assert plot_figures.main(["curves", str(log)]) == {str(log): [(0.03, 0.0244), (0.22, 0.19)]}


def test_analyze_trace(tmp_path):
    import json
    from gt_b200.bench.analyze_trace import analyze, busy_union
    ev = [dict(ph="X", cat="kernel", name="attn_fwd_async_kernel", ts=0, dur=100),
          dict(ph="X", cat="kernel", name="ncclDevKernel_AllGather", ts=50, dur=100),          # overlaps on a second stream
          dict(ph="X", cat="kernel", name="gemm_nt_gather_kernel", ts=400, dur=100),
          dict(ph="X", cat="gpu_memcpy", name="Memcpy DtoH", ts=500, dur=20),
          dict(ph="X", cat="cpu_op", name="aten::mm", ts=0, dur=10)]
    assert busy_union(ev[:3]) == 250
    p = tmp_path / "t.json"
    p.write_text(json.dumps(dict(traceEvents=ev)))
    r = analyze(str(p))
    assert r["kernels"] == 4 and abs(r["wall_ms"] - 0.52) < 1e-9 and abs(r["busy_ms"] - 0.27) < 1e-9 and r["gaps"] == 1
    assert abs(r["largest_gaps"][0]["ms"] - 0.25) < 1e-9
    assert len(r["collectives"]) == 1 and r["per_category_ms"]["attention"] == 0.1


def test_check_int32_structures():
    from gt_b200.bench.check_int32_structures import built, limits
    assert not limits(111_059_956, 3_339_184_668, 1, 1)["ok"]
    assert limits(111_059_956, 3_339_184_668, 2, 4)["ok"]
    assert limits(111_059_956, 3_339_184_668, 1, 1, stream_sub=4)["tile_edges"] > 2 ** 31         # the tile itself still overflows
    r = built("cpu_small", 2, 2)
    assert r["ok"] and r["dtypes"] == ["torch.int32"] and r["edges"] == r["max_ptr"]


def test_torchgt_batch_construction_and_cpu_run():
    import torch
    from gt_b200.bench.torchgt_batch_bench import main, torchgt_batch
    x, y = torch.randn(10, 3), torch.arange(10)
    ei = torch.tensor([[0, 1, 2, 3, 8], [1, 2, 3, 4, 9]])
    xb, yb, eb, n = torchgt_batch(x, y, ei, torch.tensor([1, 2, 3, 9]), 4, seed=0)
    assert n == 5 and xb.shape == (4, 3) and eb.shape[1] == 2 + 8           # edges 1->2, 2->3 survive; 4 token edges each way
    assert int(eb.min()) == 0 and int(eb.max()) == 4
    inner = eb[:, :2] - 1
    assert {(int(yb[s]), int(yb[d])) for s, d in inner.t()} == {(1, 2), (2, 3)}
    res = main(["--graph", "cpu_small", "--seq_len", "200", "--device", "cpu", "--iters", "1", "--warmup", "1", "--hidden", "32", "--ffn", "32",
                "--heads", "4", "--layers", "2"])
    assert res["batch_nodes"] == 200 and res["iteration_ms"] > 0


def _torchgt_worker(rank, world):
    from gt_b200.bench.torchgt_batch_bench import main
    res = main(["--graph", "cpu_small", "--seq_len", "200", "--device", "cpu", "--iters", "1", "--warmup", "1", "--hidden", "32", "--ffn", "32",
                "--heads", "4", "--layers", "2", "--grid", "2", "1", "--fused"])
    assert res["grid"] == [2, 1] and res["iteration_ms"] > 0


def test_torchgt_batch_bench_on_a_grid():
    run_dist(_torchgt_worker, 2)


# ---- GPU: the kernel studies run end to end on small cases -----------------------------------------------------------------

@pytest.mark.gpu
def test_kernel_theory_and_capture_workload_on_gpu(tmp_path):
    from gt_b200.bench import kernel_ncu, kernel_theory
    res = kernel_theory.main(["--rows", "8192", "--degrees", "0", "2", "16", "32", "--iters", "2", "--out", str(tmp_path / "t.json")])
    assert res["hbm_read_gbs"] > 1000 and len(res["sweep"]) == 4
    assert res["sweep"][3]["bwd_ms"] > 0 and res["fit"]["fwd"]["ns_per_edge"] is not None
    info = {k["name"]: k for k in res["kernels"]}
    assert info["fwd_ring_bf16_8x32"]["regs"] > 0 and info["fwd_ring_bf16_8x32"]["blocks_per_sm"] >= 4
    assert info["row_ring_bf16_8x32"]["blocks_per_sm"] >= 4 and info["col_ring_bf16_8x32"]["blocks_per_sm"] >= 4
    assert all(k["local_bytes"] == 0 for k in res["kernels"] if "ring" in k["name"])      # no array of a default kernel lives in local memory
    import torch
    from gt_b200.attention import backend_cuda as bc
    blk = kernel_theory.regular_block(512, 0).to("cuda")                                    # a tile without edges: zeros, no edge types read
    q, k, v = (torch.randn(512, 8, 32, device="cuda").bfloat16() for _ in range(3))
    acc, l, m = bc.attn_fwd_partial(q, k, v, blk, torch.randn(3, 8, 32, device="cuda"), None, score="gated", norm="clampexp")
    assert float(acc.abs().max()) == 0.0 and float(l.abs().max()) == 0.0
    order = kernel_ncu.main(["--rows", "4096", "--degrees", "1", "8", "--order", str(tmp_path / "o.json")])
    assert [c["call"] for c in order] == ["fwd", "bwd", "fwd", "bwd"]


@pytest.mark.gpu
def test_kernel_option_benches_on_gpu():
    from gt_b200.bench import bench_kernel_external, bench_kernel_opts, bench_row_overhead
    rows = bench_kernel_opts.main(["--blocks", "tile24", "--layouts", "8x32", "4x64", "--dtypes", "bf16", "fp32", "--iters", "2"])
    assert len(rows) == 4 and all(r["fwd_ms"] > 0 and r["bwd_ms"] > 0 for r in rows)
    rows = bench_row_overhead.main(["--rows", "20000", "--cols", "5000", "--per_row", "0.5", "2", "--iters", "2"])
    assert rows[0]["nonempty_rows"] < 20000 and rows[0]["fwd_accum_ms"] > 0
    rows = bench_kernel_external.main(["--graph", "cpu_small", "--layouts", "4x32", "--iters", "2"])
    by = {r["impl"]: r for r in rows}
    assert by["cuda"]["max_abs_diff_vs_edge_list"] < 0.05 and by["csr_torch"]["max_abs_diff_vs_edge_list"] < 1e-3
    assert "fwd_ms" in by["dense_sdpa"] and ("fwd_ms" in by["sparse_lib"] or "error" in by["sparse_lib"])


def test_profile_exports_a_chrome_trace_for_analyze_trace(tmp_path, monkeypatch):
    import io
    import torch
    from gt_b200.bench.analyze_trace import analyze
    from gt_b200.utils.profiling import kernel_profile
    monkeypatch.setenv("GT_PROF_TRACE", str(tmp_path / "step"))
    with kernel_profile(rank=0, file=io.StringIO()):
        torch.ones(64, 64) @ torch.ones(64, 64)
    path = tmp_path / "step_rank0.json"
    assert path.exists()
    r = analyze(str(path))
    assert r["kernels"] == 0 or r["busy_ms"] > 0            # CPU run: a valid trace without GPU events


# ---- sparse-collective diagnosis tools ------------------------------------------------------------------------------------

def test_bench_sparse_accumulate_candidates_agree():
    from gt_b200.bench.bench_sparse_accumulate import main
    res = main(["--cases", "300:1:16", "200:3:8", "--iters", "1"])
    assert len(res) == 2 and "index_copy_ms" in res[0] and "index_copy_ms" not in res[1]
    assert all(r["index_add_ms"] > 0 and r["sort_segment_ms"] > 0 for r in res)


def _profile_sparse_worker(rank, world):
    from gt_b200.bench.profile_sparse_comm import main
    res = main(["--rows", "512", "--width", "16", "--share", "0.3", "--iters", "1"])
    assert res["gather_ms"] > 0 and res["reduce_ms"] > 0 and 0.2 < res["share"] < 0.4


def test_profile_sparse_comm_on_gloo():
    run_dist(_profile_sparse_worker, 2)


def test_analyze_coll_tables(tmp_path, capsys):
    import json
    from gt_b200.bench.analyze_coll_tables import main
    a = {"_world": 4, "coll": {"rs": [20.0, 300.0]}, "_coll_curves_mb_ms": {"rs": [[1.0, 0.02], [64.0, 0.25]], "ag": [[1.0, 0.01]]}}
    b = {"_world": 8, "coll": {"rs": [30.0, 150.0]}, "_coll_curves_mb_ms": {"rs": [[64.0, 0.5]]}}
    pa, pb = tmp_path / "a.json", tmp_path / "b.json"
    pa.write_text(json.dumps(a)); pb.write_text(json.dumps(b))
    out = main([str(pa), str(pb)])
    assert set(out) == {"rs", "ag"}
    assert out["rs"]["columns"] == ["a@4", "b@8"]
    assert out["rs"]["rates"][64.0] == [round(64 * 2 ** 20 / 0.25e-3 / 1e9, 1), round(64 * 2 ** 20 / 0.5e-3 / 1e9, 1)]
    assert out["rs"]["rates"][1.0][1] is None
    assert "RS: GB/s" in capsys.readouterr().out


def test_kernel_l2_factor_arithmetic():
    from gt_b200.bench.kernel_l2 import L2_BYTES, gathered_bytes, l2_factor
    assert gathered_bytes(32768, 8, 32) == 2 * 32768 * 256 * 2 < L2_BYTES // 2
    lam = l2_factor(dict(edges=100, fwd_ms=1.0, bwd_ms=4.0), dict(edges=200, fwd_ms=4.0, bwd_ms=8.0))
    assert lam == {"fwd": 0.5, "bwd": 1.0}


def test_plot_series_time_to_accuracy_model_and_versus(tmp_path):
    import json
    from gt_b200.bench import parse_logs, plot_figures
    log = tmp_path / "a.log"
    log.write_text(
        "epoch    0 loss 3.8 train 0.02 val 0.10 test 0.02 | best val 0.10 test 0.02 @ 0 | 30.0 ms/epoch train\n"
        "epoch   10 loss 3.1 train 0.20 val 0.45 test 0.18 | best val 0.45 test 0.18 @ 10 | 20.0 ms/epoch train\n"
        "epoch   20 loss 2.9 train 0.30 val 0.55 test 0.28 | best val 0.55 test 0.28 @ 20 | 20.0 ms/epoch train\n")
    rows = parse_logs.curves([str(log)])
    tta = plot_figures.time_to_acc_series(rows, "val_acc", 0.5)
    assert list(tta) == [str(log)] and abs(tta[str(log)] - 0.42) < 1e-9
    assert plot_figures.time_to_acc_series(rows, "val_acc", 0.9) == {}
    model = plot_figures.model_series()
    assert {"world 1", "world 4", "world 8"} <= set(model)
    assert all(0.8 < p / m < 1.25 for pts in model.values() for m, p, _ in pts)
    res = tmp_path / "bench.jsonl"
    res.write_text("\n".join(json.dumps(d) for d in [
        dict(impl="reference", n_gpus=1, ms_per_step=100.0), dict(impl="gt_b200", n_gpus=1, ms_per_step=20.0),
        dict(impl="reference", n_gpus=8, ms_per_step=40.0), dict(impl="gt_b200", n_gpus=8, ms_per_step=5.0),
        dict(impl="gt_b200", n_gpus=4, ms_per_step=9.0)]) + "\nnot json\n")
    assert plot_figures.main(["versus", str(res)]) == {"speed-up over reference": [(1, 5.0), (8, 8.0)]}
    assert plot_figures.main(["time_to_acc", str(log), "--target", "0.5"]) == tta


def test_tile_density_orders():
    import torch
    from gt_b200.bench import tile_density as td
    n = 1024
    blocks = [torch.cartesian_prod(torch.arange(b * 128, (b + 1) * 128), torch.arange(b * 128, (b + 1) * 128)).t() for b in range(4)]
    dense = torch.cat(blocks, 1)                                     # four fully dense diagonal tiles
    dense = dense[:, torch.rand(dense.shape[1], generator=torch.Generator().manual_seed(0)) < 0.5]
    st = td.tile_stats(dense, n, 1638)
    assert st["dense_tiles"] == 4 and st["dense_edge_share"] == 1.0 and st["tiles_nonempty"] == 4 and st["tiles_total"] == 64
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(1))
    assert td.tile_stats(perm[dense], n, 1638)["dense_edge_share"] == 0.0      # a random relabelling destroys the tiles
    star = torch.stack([torch.full((600,), 900), torch.arange(600)])            # node 900 is the hub
    ei = td.degree_order(torch.cat([star, star.flip(0)], 1), n)
    assert int(ei[0][0]) == 0                                         # the hub becomes node 0
    res = td.main(["--graph", "cpu_small", "--orders", "native", "degree", "--min_edges", "64"])
    assert [r["order"] for r in res] == ["native", "degree"] and all(r["edges"] > 0 for r in res)


def test_curves_from_metrics_jsonl(tmp_path):
    import json
    from gt_b200.bench import parse_logs, plot_figures
    f = tmp_path / "m.jsonl"
    f.write_text("\n".join(json.dumps(dict(epoch=e, loss=3.0 - e * 0.1, train=0.1 * e, val=0.2 * e, test=0.15 * e, epoch_ms=20.0, best_val=0.2 * e,
                                           best_epoch=e, world=1, grid=[1, 1])) for e in (0, 2, 4)) + "\n")
    rows = parse_logs.curves_jsonl([str(f)])
    assert [r["epoch"] for r in rows] == [0, 2, 4] and abs(rows[-1]["train_seconds"] - 0.1) < 1e-9
    assert plot_figures.time_to_acc_series(rows, "val_acc", 0.4) == {str(f): rows[1]["train_seconds"]}


def _bench_modules():
    import glob
    import os
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "gt_b200", "bench")
    names = sorted(os.path.basename(f)[:-3] for f in glob.glob(os.path.join(root, "*.py")))
    return [n for n in names if not n.startswith("_") and n != "model_validation_data"]


def test_every_bench_tool_imports_and_answers_help_without_a_gpu():
    """The measurement tools need GPUs to measure, but none may need one to import or to print its usage."""
    import subprocess
    import sys
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = {n: subprocess.Popen([sys.executable, "-m", f"gt_b200.bench.{n}", "--help"], cwd=root, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
             for n in _bench_modules()}
    assert len(procs) >= 25
    for n, p in procs.items():
        out, _ = p.communicate(timeout=300)
        assert p.returncode == 0 and len(out) > 40, (n, p.returncode, out[-300:])


def test_timing_regression_check(tmp_path, capsys):
    import json
    from gt_b200.bench import check_regression as cr
    assert cr.recorded_ms((4, 2)) == 6.00 and cr.recorded_ms((3, 3)) is None
    line = dict(ms_per_step=6.2, config=dict(grid=[4, 2]), clocks=dict(reasons=[]))
    assert cr.assess(line)[0] == "ok"
    assert cr.assess(dict(line, ms_per_step=7.5))[0] == "slower"
    assert cr.assess(dict(line, ms_per_step=9.0, clocks=dict(reasons=["sw_thermal_slowdown"])))[0] == "inconclusive"
    assert cr.assess(dict(line, clocks=dict(reasons=["sw_power_cap"])))[0] == "ok"          # a power cap during dense kernels is normal
    assert cr.assess(dict(line, config=dict(grid=[3, 3])))[0] == "unknown"
    assert cr.assess(dict(line, ms_per_step=40.6, impl="reference"))[0] == "unknown"       # the reference arm's lines are not compared
    assert cr.assess(dict(ms_per_step=27.0, config=dict(parallelism="grid 1x1")))[0] == "slower"
    f = tmp_path / "lines.txt"
    f.write_text("NCCL version 2.28\n" + json.dumps(line) + "\n" + json.dumps(dict(line, ms_per_step=19.0, config=dict(grid=[1, 1]))) + "\n")
    assert cr.main(["--from_json", str(f)]) == 0
    out = capsys.readouterr().out
    assert "[ok] grid 4x2" in out and "[ok] grid 1x1" in out
    g = tmp_path / "slow.json"
    g.write_text(json.dumps(dict(line, ms_per_step=8.0)))
    assert cr.main(["--from_json", str(g), "--tolerance", "0.2"]) == 1


def test_every_module_of_the_package_imports_without_a_gpu():
    import importlib
    import pkgutil
    import gt_b200
    bad = []
    for m in pkgutil.walk_packages(gt_b200.__path__, "gt_b200."):
        try:
            importlib.import_module(m.name)
        except Exception as exc:                             # noqa: BLE001
            bad.append((m.name, repr(exc)[:200]))
    assert not bad, bad
