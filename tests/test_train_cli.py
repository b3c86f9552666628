"""The ``train_dist`` command line end to end on CPU (single process and gloo ranks), checkpoint save / resume, and the
observability switches."""
import os

import pytest
import torch

from dist_utils import run_dist


def _run(argv):
    from gt_b200.train.train_dist import main
    return main(argv)


def test_single_process_trains_and_resumes(tmp_path, capsys):
    ck = str(tmp_path / "ck.pt")
    base = ["--synthetic", "cpu_small", "--scale_down", "4", "--fused", "--norm", "ln", "--lr", "5e-3", "--dropout", "0.0", "--warmup", "1"]
    _run(base + ["--epochs", "6", "--save", ck, "--save_every", "3"])
    out = capsys.readouterr().out
    assert "data: N=" in out and "FINAL best_val=" in out and "STEADY model=exphormer" in out and "ms_per_epoch=" in out
    blob = torch.load(ck, map_location="cpu", weights_only=False)
    assert blob["epoch"] == 6 and "optimizer" in blob and "layers.0.q.weight" in blob["model"]


def test_resume_matches_uninterrupted(tmp_path):
    from gt_b200.train import train_dist
    ck = str(tmp_path / "half.pt")
    base = ["--synthetic", "cpu_small", "--scale_down", "4", "--fused", "--norm", "ln", "--dropout", "0.0", "--warmup", "1", "--lr", "5e-3"]
    full = train_dist.main(base + ["--epochs", "6", "--save", str(tmp_path / "full.pt")])
    # first half: the schedule must be the 6-epoch one, so run 6 epochs' schedule but stop at 3 via save_every and reload that file
    train_dist.main(base + ["--epochs", "6", "--save", ck, "--save_every", "3"])
    a = torch.load(str(tmp_path / "full.pt"), weights_only=False)["model"]
    b = torch.load(ck, weights_only=False)["model"]
    for k in a:
        assert torch.equal(a[k], b[k]), k                       # same seed, same run: deterministic on CPU
    # now interrupt for real: save at epoch 3, resume to 6
    part = str(tmp_path / "part.pt")

    class Stop(Exception):
        pass
    import gt_b200.train.checkpoint as cp
    orig = cp.save_checkpoint

    def save_then_stop(path, model, engine, epoch, extra=None):
        orig(path, model, engine, epoch, extra)
        if epoch == 3:
            raise Stop()
    cp.save_checkpoint = save_then_stop
    try:
        with pytest.raises(Stop):
            train_dist.main(base + ["--epochs", "6", "--save", part, "--save_every", "3"])
    finally:
        cp.save_checkpoint = orig
    train_dist.main(base + ["--epochs", "6", "--resume", part, "--save", part])
    c = torch.load(part, weights_only=False)["model"]
    for k in a:
        assert (a[k] - c[k]).abs().max() < 1e-6, k


def _cli_worker(rank, world, argv):
    from gt_b200.train.train_dist import main
    res = main(argv)
    assert len(res["epoch_ms"]) >= 3 and res["best"]["val"] >= 0.0


@pytest.mark.parametrize("argv", [
    ["--grid", "2", "1", "--synthetic", "cpu_small", "--scale_down", "4", "--fused", "--epochs", "3", "--norm", "ln", "--coll_stats", "--timers",
     "--heartbeat", "30"],
    ["--grid", "1", "2", "--synthetic", "cpu_small", "--scale_down", "4", "--stream_sub", "2", "--fused", "--epochs", "3", "--saved_census"],
    ["--grid", "2", "1", "--synthetic", "cpu_small", "--scale_down", "4", "--model", "unimp", "--label_input", "--epochs", "3"],
    ["--grid", "1", "1", "2", "--synthetic", "cpu_small", "--scale_down", "4", "--model", "graphormer", "--epochs", "3", "--heads", "4"],
    ["--grid_auto", "--synthetic", "cpu_small", "--scale_down", "4", "--epochs", "3", "--auto_ckpt"],
    ["--grid", "2", "1", "--synthetic", "exphormer_rmat26", "--scale_down", "32768", "--stream_gen", "--stream_sub", "2", "--fused", "--epochs", "3",
     "--hidden", "32", "--heads", "4", "--norm", "ln"],
], ids=["fused_2x1_stats", "streamed_1x2_census", "unimp_label", "graphormer_head", "grid_auto", "rmat_stream_gen"])
def test_cli_on_gloo_ranks(argv):
    run_dist(_cli_worker, 2, argv)


def test_partition_directory_input(tmp_path):
    from gt_b200.data.partition import partition_2d
    from gt_b200.data.synthetic import workload_graph
    wl = workload_graph("cpu_small", scale_down=4)
    partition_2d(wl["x"], wl["y"], wl["masks"], wl["edge_index"], 10, str(tmp_path / "p2"), p_part=2)
    run_dist(_cli_worker, 2, ["--grid", "2", "1", "--data", str(tmp_path / "p2"), "--fused", "--epochs", "3", "--hidden", "32", "--heads", "4",
                              "--layers", "2"])


def test_single_gpu_trainer_learns_on_cpu(tmp_path, capsys):
    from gt_b200.train.train_single_gpu import main
    best = main(["--synthetic", "cpu_small", "--scale_down", "4", "--epochs", "12", "--hidden", "32", "--heads", "4", "--layers", "2",
                 "--lr", "1e-2", "--dropout", "0.0"])
    assert "FINAL backend=torch" in capsys.readouterr().out and best["epoch"] >= 0
    # a saved graph file goes through the same path
    g = dict(x=torch.randn(50, 8), y=torch.randint(0, 3, (50,)), edge_index=torch.randint(0, 50, (2, 120)),
             train_idx=torch.arange(0, 30), valid_idx=torch.arange(30, 40), test_idx=torch.arange(40, 50))
    torch.save(g, str(tmp_path / "g.pt"))
    main(["--graph", str(tmp_path / "g.pt"), "--epochs", "2", "--hidden", "16", "--heads", "2", "--layers", "1", "--backend", "ref"])


def test_collective_census_counts_the_peer_memory_transport(monkeypatch):
    """``CollectiveStats`` patches the symmetric heap's methods like it patches ``torch.distributed``."""
    import types
    import torch
    from gt_b200.parallel.symm import SymmetricHeap
    from gt_b200.utils.collstats import CollectiveStats
    monkeypatch.setattr(SymmetricHeap, "all_gather", lambda self, x, group: x.repeat(2, 1))
    monkeypatch.setattr(SymmetricHeap, "all_reduce", lambda self, x, out, name=None, group=None: out.copy_(2 * x))
    monkeypatch.setattr(SymmetricHeap, "pull_gather", lambda self, x2, plan: x2[:3])
    heap = SymmetricHeap.__new__(SymmetricHeap)
    heap.ctx = lambda group: types.SimpleNamespace(size=4 if group == "row" else 2)
    plain = SymmetricHeap.all_gather
    st = CollectiveStats()
    for _ in range(2):
        st.begin_epoch()
        assert heap.all_gather(torch.ones(4, 4), "row").shape == (8, 4)
        heap.all_reduce(torch.ones(8), torch.empty(8), "grads")
        heap.pull_gather(torch.ones(5, 2), types.SimpleNamespace(group=None))
        st.end_epoch()
    assert SymmetricHeap.all_gather is plain                                   # patches are removed after every epoch
    t = st.table()
    assert t[("p2p_all_gather", 4)] == dict(calls=1.0, mbytes=64 / 2 ** 20, ms=0.0)
    assert t[("p2p_all_reduce", 2)]["calls"] == 1.0 and t[("p2p_sparse_gather", 2)]["mbytes"] == 40 / 2 ** 20


def test_resilient_launcher_restarts_and_gives_up(tmp_path):
    """The supervisor resumes from the checkpoint of an earlier run and stops after MAX_RESTARTS failed attempts."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = os.path.join(root, "launch", "train_resilient.sh")
    ck = str(tmp_path / "run.pt")
    base = ["--grid", "1", "1", "--synthetic", "cpu_small", "--scale_down", "8", "--fused", "--hidden", "16", "--heads", "2", "--layers", "1"]
    env = dict(os.environ, SAVE_EVERY="2", RESTART_DELAY="0", MAX_RESTARTS="1")
    r = subprocess.run([script, "0", ck] + base + ["--epochs", "2"], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and os.path.exists(ck) and "finished after 0 restart" in r.stdout
    r = subprocess.run([script, "0", ck] + base + ["--epochs", "4"], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "continuing at epoch 2" in r.stdout
    r = subprocess.run([script, "0", str(tmp_path / "none.pt"), "--no_such_flag"], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode != 0 and "restart 1 of 1" in r.stderr and "giving up after 1 restarts" in r.stderr


def test_eval_only_reports_the_checkpoint(tmp_path, capsys):
    from gt_b200.train import train_dist
    ck = str(tmp_path / "m.pt")
    base = ["--grid", "1", "1", "--synthetic", "cpu_small", "--scale_down", "8", "--fused", "--hidden", "16", "--heads", "2", "--layers", "1"]
    trained = train_dist.main(base + ["--epochs", "3", "--save", ck, "--eval_every", "1"])
    capsys.readouterr()
    res = train_dist.main(base + ["--resume", ck, "--eval_only"])
    out = capsys.readouterr().out
    assert "EVAL checkpoint=" in out and res["epoch"] == 3
    assert abs(res["eval"]["valid"] - trained["best"]["val"]) < 0.2 and 0.0 <= res["eval"]["test"] <= 1.0
    with pytest.raises(SystemExit):
        train_dist.main(base + ["--eval_only"])


def _predict_worker(rank, world, ck, out):
    from gt_b200.train.train_dist import main
    base = ["--grid", "2", "1", "--synthetic", "cpu_small", "--scale_down", "8", "--fused", "--hidden", "16", "--heads", "2", "--layers", "1"]
    main(base + ["--epochs", "2", "--save", ck])
    res = main(base + ["--resume", ck, "--eval_only", "--predict_out", out])
    assert 0.0 <= res["eval"]["train"] <= 1.0


def test_eval_only_writes_predictions_in_node_order(tmp_path):
    ck, out = str(tmp_path / "m.pt"), str(tmp_path / "pred.pt")
    run_dist(_predict_worker, 2, ck, out)
    blob = torch.load(out, weights_only=True)
    n = blob["num_nodes"]
    assert blob["pred"].shape == (n,) and int(blob["pred"].min()) >= 0 and n == 250


def test_config_file_supplies_defaults_and_flags_win(tmp_path):
    from gt_b200.train.train_dist import build_parser, parse_with_config
    cfg = tmp_path / "run.yaml"
    cfg.write_text("grid: [2, 1]\nfused: true\nhidden: 64\n--epochs: 7\nsynthetic: cpu_small\n")
    args = parse_with_config(build_parser(), ["--config", str(cfg), "--hidden", "32"])
    assert args.grid == [2, 1] and args.fused and args.hidden == 32 and args.epochs == 7 and args.synthetic == "cpu_small"
    js = tmp_path / "run.json"
    js.write_text('{"layers": 3, "norm": "ln"}')
    args = parse_with_config(build_parser(), ["--config", str(js)])
    assert args.layers == 3 and args.norm == "ln" and args.grid == [1, 1]
    bad = tmp_path / "bad.yaml"
    bad.write_text("hiden: 64\n")
    with pytest.raises(SystemExit):
        parse_with_config(build_parser(), ["--config", str(bad)])


def test_metrics_jsonl(tmp_path):
    import json
    from gt_b200.train import train_dist
    mf = tmp_path / "m.jsonl"
    train_dist.main(["--grid", "1", "1", "--synthetic", "cpu_small", "--scale_down", "8", "--fused", "--hidden", "16", "--heads", "2", "--layers", "1",
                     "--epochs", "4", "--eval_every", "2", "--metrics_jsonl", str(mf)])
    rows = [json.loads(l) for l in mf.read_text().splitlines()]
    assert [r["epoch"] for r in rows] == [0, 2, 3] and all(r["epoch_ms"] > 0 and 0 <= r["val"] <= 1 for r in rows)
    assert rows[-1]["best_val"] >= rows[0]["val"] and rows[0]["grid"] == [1, 1]


def _p2p_worker(rank, world, argv, out_path):
    """The same run on gloo collectives and on the peer-memory transport (emulated between the CPU ranks): the losses agree."""
    from gt_b200.train.train_dist import main
    a = main(argv + ["--metrics_jsonl", out_path + ".gloo"])
    b = main(argv + ["--comm", "p2p", "--heap_mb", "64", "--check_protocol", "--metrics_jsonl", out_path + ".p2p"])
    assert len(a["epoch_ms"]) == len(b["epoch_ms"])
    assert abs(a["best"]["val"] - b["best"]["val"]) < 1e-6


@pytest.mark.parametrize("argv", [
    ["--grid", "2", "2", "--synthetic", "cpu_small", "--scale_down", "4", "--fused", "--epochs", "4", "--norm", "ln", "--dropout", "0.0"],
    ["--grid", "2", "2", "--synthetic", "cpu_small", "--scale_down", "4", "--fused", "--epochs", "4", "--sparse_comm", "--sparse_threshold", "1.0",
     "--dropout", "0.0"],
    ["--grid", "2", "1", "2", "--synthetic", "cpu_small", "--scale_down", "4", "--no_gcn", "--epochs", "4", "--heads", "4", "--dropout", "0.0"],
], ids=["fused_2x2", "sparse_2x2", "head_2x1x2"])
def test_cli_comm_p2p_between_cpu_ranks_matches_gloo(argv, tmp_path):
    import json
    out = str(tmp_path / "m")
    run_dist(_p2p_worker, 4, argv, out)
    rows = {k: [json.loads(line) for line in open(out + "." + k)] for k in ("gloo", "p2p")}
    assert len(rows["gloo"]) == len(rows["p2p"]) > 0
    for ra, rb in zip(rows["gloo"], rows["p2p"]):
        assert abs(ra["loss"] - rb["loss"]) < 1e-4 * max(1.0, abs(ra["loss"])), (ra, rb)


def _token_dense_cli_worker(rank, world, out_path):
    from gt_b200.train.train_dist import main
    base = ["--grid", "2", "2", "--synthetic", "cpu_small", "--scale_down", "4", "--fused", "--virtual_node", "--epochs", "4", "--norm", "ln",
            "--dropout", "0.0"]
    main(base + ["--metrics_jsonl", out_path + ".edges"])
    main(base + ["--token_dense", "--metrics_jsonl", out_path + ".dense"])
    with pytest.raises(SystemExit):
        main(["--grid", "2", "2", "--synthetic", "cpu_small", "--token_dense", "--epochs", "1"])


def test_cli_token_dense_trains_like_token_edges(tmp_path):
    import json
    out = str(tmp_path / "m")
    run_dist(_token_dense_cli_worker, 4, out)
    rows = {k: [json.loads(line) for line in open(out + "." + k)] for k in ("edges", "dense")}
    assert len(rows["edges"]) == len(rows["dense"]) > 0
    for ra, rb in zip(rows["edges"], rows["dense"]):
        assert abs(ra["loss"] - rb["loss"]) < 1e-4 * max(1.0, abs(ra["loss"])), (ra, rb)


def test_launch_scripts_parse_and_never_touch_gpu_settings():
    """Shell syntax of every launcher; none of them sets clocks, power limits, persistence or compute modes, and every Nsight Compute
    command line leaves the clocks alone."""
    import glob
    import re
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    scripts = sorted(glob.glob(os.path.join(root, "launch", "*")) + [os.path.join(root, "baseline", "dac26", "launch.sh")])
    assert len(scripts) >= 8
    for path in scripts:
        assert subprocess.run(["bash", "-n", path]).returncode == 0, path
        text = open(path).read()
        assert not re.search(r"nvidia-smi\s+(-lgc|-ac|-pm|-pl|-c|--lock|--reset|-rgc|-r\b)", text), path
        for line in text.splitlines():
            if re.match(r"\s*ncu\s", line) or " ncu " in line and not line.lstrip().startswith("#"):
                assert "--clock-control none" in text, path


def _two_machines_cli_worker(rank, world):
    os.environ["GT_HOSTNAME"] = "node%d" % (rank // 2)
    try:
        from gt_b200.train.train_dist import main
        res = main(["--grid", "2", "2", "--synthetic", "cpu_small", "--scale_down", "4", "--fused", "--epochs", "3", "--norm", "ln", "--comm", "p2p",
                    "--heap_mb", "64", "--check_protocol"])
        assert len(res["epoch_ms"]) == 3
    finally:
        os.environ.pop("GT_HOSTNAME", None)


def test_cli_on_two_pretended_machines_mixes_the_transports(capfd):
    run_dist(_two_machines_cli_worker, 4)
    out = capfd.readouterr().out
    assert "[comm] 2 machines: row group on peer memory, column group on NCCL, gradient all-reduce on NCCL" in out
    assert "[protocol]" in out


def test_resilient_launcher_retries_an_out_of_memory_run_with_checkpointing(tmp_path):
    """A stand-in interpreter fails the first attempt with an out-of-memory message; the supervisor's second attempt carries --checkpoint."""
    import stat
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    fake = tmp_path / "fakepython"
    calls = tmp_path / "calls.txt"
    fake.write_text(f"""#!/usr/bin/env bash
echo "$@" >> {calls}
if [ "$(wc -l < {calls})" -eq 1 ]; then echo "torch.OutOfMemoryError: CUDA out of memory. Tried to allocate 20.00 GiB" >&2; exit 1; fi
exit 0
""")
    fake.chmod(fake.stat().st_mode | stat.S_IXUSR)
    env = dict(os.environ, PYTHON=str(fake), RESTART_DELAY="0", MAX_RESTARTS="2")
    r = subprocess.run([os.path.join(root, "launch", "train_resilient.sh"), "0", str(tmp_path / "x.pt"), "--grid", "1", "1"], env=env, capture_output=True,
                       text=True, timeout=120)
    lines = calls.read_text().splitlines()
    assert r.returncode == 0 and len(lines) == 2, (r.stdout, r.stderr)
    assert "--checkpoint" not in lines[0] and "--checkpoint" in lines[1]
    assert "ran out of memory" in r.stderr and "finished after 1 restart" in r.stdout


def _regrid_worker(rank, world, tmp):
    """A checkpoint does not depend on the grid: saved on 2 x 1, resumed on 1 x 2, the run continues like the uninterrupted one."""
    from gt_b200.train.train_dist import main
    base = ["--synthetic", "cpu_small", "--scale_down", "4", "--fused", "--norm", "ln", "--dropout", "0.0", "--warmup", "1", "--lr", "5e-3", "--epochs", "6"]
    main(["--grid", "2", "1"] + base + ["--metrics_jsonl", tmp + "/full.jsonl"])
    ck = tmp + "/half.pt"

    class Stop(Exception):
        pass
    from gt_b200.train import checkpoint as cp
    real = cp.save_checkpoint

    def save_then_stop(path, model, eng, epoch, extra=None):
        real(path, model, eng, epoch, extra)
        if epoch == 3:
            raise Stop()
    cp.save_checkpoint = save_then_stop
    try:
        with pytest.raises(Stop):
            main(["--grid", "2", "1"] + base + ["--save", ck, "--save_every", "3"])
    finally:
        cp.save_checkpoint = real
    import torch.distributed as dist
    dist.barrier()
    main(["--grid", "1", "2"] + base + ["--resume", ck, "--metrics_jsonl", tmp + "/resumed.jsonl"])


def test_checkpoint_resumes_on_another_grid(tmp_path):
    import json
    run_dist(_regrid_worker, 2, str(tmp_path))
    full = [json.loads(line) for line in open(tmp_path / "full.jsonl")]
    res = [json.loads(line) for line in open(tmp_path / "resumed.jsonl")]
    assert [r["epoch"] for r in res] == [3, 4, 5] or res[-1]["epoch"] == 5
    last_full = [r for r in full if r["epoch"] == 5][0]
    last_res = [r for r in res if r["epoch"] == 5][0]
    assert abs(last_full["loss"] - last_res["loss"]) < 1e-4 * max(1.0, abs(last_full["loss"])), (last_full, last_res)


def test_nccl_tune_only_touches_the_environment_when_the_column_group_crosses_machines(monkeypatch):
    from gt_b200.train import train_dist as td
    for var in ("NCCL_ALGO", "NCCL_MIN_NCHANNELS"):
        monkeypatch.delenv(var, raising=False)
    parse = td.build_parser().parse_args
    monkeypatch.setenv("WORLD_SIZE", "8"); monkeypatch.setenv("LOCAL_WORLD_SIZE", "8")
    assert "NCCL defaults" in td.nccl_tune(parse(["--grid", "4", "2"])) and "NCCL_ALGO" not in os.environ
    monkeypatch.setenv("WORLD_SIZE", "32")
    assert "NCCL defaults" in td.nccl_tune(parse(["--grid", "4", "8", "--sparse_comm"])) and "NCCL_ALGO" not in os.environ
    assert td.nccl_tune(parse(["--grid", "4", "8", "--nccl_tune", "off"])) is None
    line = td.nccl_tune(parse(["--grid", "4", "8"]))
    assert "4 machine(s)" in line and os.environ["NCCL_ALGO"] == "Ring" and os.environ["NCCL_MIN_NCHANNELS"] == "16"
    monkeypatch.delenv("NCCL_ALGO"); monkeypatch.delenv("NCCL_MIN_NCHANNELS")
    monkeypatch.setenv("WORLD_SIZE", "8")
    assert "NCCL_ALGO=Ring" in td.nccl_tune(parse(["--grid", "4", "2", "--nccl_tune", "on"]))
    monkeypatch.delenv("NCCL_ALGO"); monkeypatch.delenv("NCCL_MIN_NCHANNELS")
