"""Host-only pieces: the 5-D rank grid arithmetic, the data loader's data-parallel sampling and
context-parallel slicing, the utilities, and the tools around the trainer (metrics extraction, Slurm
job rendering and status files)."""
import json
import os
import sys
import types

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


# ---------------------------------------------------------------------------------------------
# rank grid (picotron/process_group_manager.py:24-30: grid = arange(world).view(dp, pp, cp, ep, tp))
# ---------------------------------------------------------------------------------------------
def test_grid_matches_arange_view_and_groups_partition_the_world():
    from picotron_b200.process_group_manager import AXES, GridTopology
    g = GridTopology(tp=2, cp=2, pp=3, dp=2, ep=2)
    assert g.world_size == 48 and g.shape == (2, 3, 2, 2, 2)
    grid = torch.arange(g.world_size).view(*g.shape)
    for rank in range(g.world_size):
        c = g.coords(rank)
        assert grid[c["dp"], c["pp"], c["cp"], c["ep"], c["tp"]].item() == rank
        assert g.rank_of(**c) == rank
    # tensor-parallel ranks are adjacent, data-parallel ranks are the farthest apart
    assert g.group_ranks(0, ("tp",)) == [0, 1]
    assert g.group_ranks(0, ("dp",)) == [0, 24]
    for axis in AXES:
        groups = g.all_groups((axis,))
        flat = sorted(r for grp in groups for r in grp)
        assert flat == list(range(g.world_size)), axis            # a partition of the world
        assert all(len(grp) == dict(zip(AXES, g.shape))[axis] for grp in groups)
    # the gradient-sync group spans cp and dp but never ep (process_group_manager.py:78-89)
    cp_dp = g.group_ranks(5, ("cp", "dp"))
    assert len(cp_dp) == 4 and all(g.coords(r)["ep"] == g.coords(5)["ep"] for r in cp_dp)
    assert all(g.coords(r)["tp"] == g.coords(5)["tp"] and g.coords(r)["pp"] == g.coords(5)["pp"] for r in cp_dp)


def test_grid_rejects_out_of_range_coordinates():
    from picotron_b200.process_group_manager import GridTopology
    g = GridTopology(tp=2, dp=2)
    with pytest.raises(AssertionError):
        g.rank_of(dp=0, pp=0, cp=0, ep=0, tp=2)
    with pytest.raises(AssertionError):
        g.coords(4)


# ---------------------------------------------------------------------------------------------
# data loader (picotron/data.py:33-36,59-64,112-123)
# ---------------------------------------------------------------------------------------------
def _loader(dp, dp_rank, cp, cp_rank, **kw):
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.data import MicroBatchDataLoader
    pgm.process_group_manager = types.SimpleNamespace(dp_world_size=dp, dp_rank=dp_rank, cp_world_size=cp,
                                                      cp_rank=cp_rank)
    try:
        return MicroBatchDataLoader(micro_batch_size=2, seq_length=16, dataset_name="synthetic", grad_acc_steps=3,
                                    num_samples=64, vocab_size=100, seed=7, pin_memory=False, **kw)
    finally:
        pgm.process_group_manager = None


def test_loader_shapes_and_context_parallel_slices_tile_the_sequence():
    full = next(_loader(1, 0, 1, 0))
    assert full["input_ids"].shape == (2, 16) and full["hidden_states"] is None
    assert torch.equal(full["input_ids"][:, 1:], full["target_ids"][:, :-1])       # targets = inputs shifted by one
    parts = [next(_loader(1, 0, 4, r)) for r in range(4)]
    assert all(p["input_ids"].shape == (2, 4) for p in parts)
    assert torch.equal(torch.cat([p["input_ids"] for p in parts], dim=1), full["input_ids"])
    assert torch.equal(torch.cat([p["target_ids"] for p in parts], dim=1), full["target_ids"])
    assert torch.equal(torch.cat([p["position_ids"] for p in parts], dim=1), full["position_ids"])
    ld = _loader(2, 1, 2, 0)
    assert (ld.global_batch_size, ld.num_global_micro_batches, ld.seq_length_per_gpu) == (12, 6, 8)


def test_loader_data_parallel_ranks_take_interleaved_samples_and_resume():
    a, b = _loader(2, 0, 1, 0), _loader(2, 1, 1, 0)
    single = _loader(1, 0, 1, 0)
    first = next(single)["input_ids"], next(single)["input_ids"]        # samples 0,1 then 2,3
    ra, rb = next(a)["input_ids"], next(b)["input_ids"]                  # rank 0: samples 0,2; rank 1: samples 1,3
    assert torch.equal(ra[0], first[0][0]) and torch.equal(rb[0], first[0][1])
    assert torch.equal(ra[1], first[1][0]) and torch.equal(rb[1], first[1][1])
    state = a.state_dict()
    expected = next(a)["input_ids"]
    fresh = _loader(2, 0, 1, 0)
    fresh.load_state_dict(state)
    assert torch.equal(next(fresh)["input_ids"], expected)


# ---------------------------------------------------------------------------------------------
# utilities (picotron/utils.py:35-62)
# ---------------------------------------------------------------------------------------------
def test_readable_format_and_mfu_formula():
    from picotron_b200 import utils
    assert utils.to_readable_format(1234).endswith("K") and utils.to_readable_format(2.5e9).endswith("B")
    assert utils.to_readable_format(12) == "12" or utils.to_readable_format(12).startswith("12")
    n, L, h, s = 1.7e9, 24, 2048, 2048
    fpt = utils.flops_per_token(n, L, h, s)
    assert fpt == pytest.approx(6 * n + 12 * L * h * s)
    cfg = types.SimpleNamespace(num_hidden_layers=L, hidden_size=h, max_position_embeddings=s)
    mfu = utils.get_mfu(10000.0, n, cfg, theoretical_flops=989.5e12) if "theoretical_flops" in \
        utils.get_mfu.__code__.co_varnames else None
    if mfu is not None:
        assert mfu == pytest.approx(10000.0 * fpt / 989.5e12 * 100, rel=1e-6)


# ---------------------------------------------------------------------------------------------
# metrics extractor (extract_metrics.py of the reference: :10-25 folder names, :54-87 log lines)
# ---------------------------------------------------------------------------------------------
def _write_log(path, steps):
    with open(path, "w") as fh:
        fh.write("some banner line\n")
        for i, (tok, mfu) in enumerate(steps, start=1):
            fh.write(f"[default0]:[rank 0] Step: {i:<5d} | Loss: 10.1 | Global batch size: 524.3K | "
                     f"Tokens/s: 80.0K | Tokens/s/GPU: {tok} | Tokens: 1.0M | MFU: {mfu}% | Memory usage: 10.0MB\n")


def test_extract_metrics_parses_names_and_skips_warmup(tmp_path):
    import extract_metrics as em
    p = em.parse_folder_name("dp2_tp4_pp1_mbs4_ga8_sl2048")
    assert (p["dp"], p["tp"], p["pp"], p["mbs"], p["ga"], p["sl"]) == (2, 4, 1, 4, 8, 2048) and p["ep"] is None
    assert em.parse_folder_name("dp1_tp1_pp1_cp2_ep8_mbs1_ga1_sl4096")["ep"] == 8
    run = tmp_path / "dp2_tp4_pp1_mbs4_ga8_sl2048"
    run.mkdir()
    steps = [("1.0K", "1.0"), ("2.0K", "2.0"), ("3.0K", "3.0"), ("40.0K", "40.0"), ("60.0K", "50.0")]
    _write_log(run / "log_1.out", steps)
    status, tok, mfu = em.process_run(str(run))
    assert status == "completed"
    assert tok == pytest.approx(50000.0) and mfu == pytest.approx(45.0)      # steps 1-3 are warm-up
    assert (run / "metrics.csv").exists()
    (run / "status.txt").write_text("oom")
    assert em.process_run(str(run))[0] == "oom"
    empty = tmp_path / "dp1_tp1_pp1_mbs1_ga1_sl128"
    empty.mkdir()
    assert em.process_run(str(empty)) == ("unknown", None, None)


# ---------------------------------------------------------------------------------------------
# Slurm scheduler (submit_slurm_jobs.py of the reference: :9-57 status file, :83-92 world size)
# ---------------------------------------------------------------------------------------------
def _job_dir(root, name, **dist):
    d = root / name
    d.mkdir(parents=True)
    cfg = {"distributed": dict(tp_size=1, cp_size=1, pp_size=1, dp_size=1, ep_size=1)}
    cfg["distributed"].update(dist)
    (d / "config.json").write_text(json.dumps(cfg))
    return d


def test_slurm_status_machine_world_size_and_rendering(tmp_path, capsys):
    pytest.importorskip("jinja2")
    import submit_slurm_jobs as ssj
    a = _job_dir(tmp_path, "a", tp_size=4, dp_size=2)
    b = _job_dir(tmp_path, "b", ep_size=8, dp_size=2)
    sch = ssj.Scheduler(str(tmp_path), qos="normal")
    assert sorted(j.name for j in sch.jobs) == ["a", "b"]
    assert all(j.status == ssj.Status.INIT for j in sch.jobs) and (a / "status.txt").read_text() == "init"
    jobs = {j.name: j for j in sch.jobs}
    assert jobs["a"].world_size() == 8
    assert jobs["b"].world_size() == 16                      # expert parallelism counts towards the world size
    script = sch.render(jobs["b"])
    text = open(script).read()
    assert "--nodes=2" in text.replace(" ", "").replace("#SBATCH", "") or "nodes=2" in text.replace(" ", "")
    assert str(b / "config.json") in text
    jobs["a"].set_status(ssj.Status.FAIL)
    again = ssj.Scheduler(str(tmp_path), qos="normal")
    assert [j.name for j in again.select()] == ["b"]         # only untouched jobs by default
    assert [j.name for j in again.select(only="fail")] == ["a"]
    assert again.summary() == {"fail": 1, "init": 1}
    again.submit(again.select(), nb_chains=1, dry_run=True)
    assert "sbatch --parsable" in capsys.readouterr().out
    (a / "status.txt").write_text("garbage")
    assert ssj.Job(str(a), "normal").status == ssj.Status.INIT
