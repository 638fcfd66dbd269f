"""Multi-process tests on CPU ranks (TCP mesh + shared-memory windows), 4 ranks on this host.
The same cases run on GPUs in tests/test_gpu_multi.py."""
import os

import pytest

from conftest import run_ranks


@pytest.mark.parametrize("case", ["basics", "collectives", "neighbor_ops", "windows", "errors",
                                  "skip_negotiate", "optimizers"])
def test_case_4_ranks(case):
    run_ranks(case, 4)


def test_basics_single_rank():
    run_ranks("basics", 1)


def test_collectives_three_ranks():
    run_ranks("collectives", 3)


def test_hierarchical_two_fake_machines():
    run_ranks("hierarchical", 4, env={"BLUEFOG_NODES_PER_MACHINE": "2"})


def test_average_consensus_config():
    out = run_ranks("consensus", 4, timeout=400)
    assert "consensus deviations" in out[0][1]


def test_timeline_files(tmp_path):
    prefix = str(tmp_path / "tl_")
    run_ranks("timeline", 2, env={"BLUEFOG_TIMELINE": prefix})
    assert os.path.exists(prefix + "0.json") and os.path.exists(prefix + "1.json")


def test_checkpoint_roundtrip(tmp_path):
    run_ranks("checkpoint", 2, env={"BFB_CKPT": str(tmp_path / "ckpt.pth.tar")})


def test_checkpoint_found_on_the_root_only(tmp_path):
    run_ranks("checkpoint_root_only", 3, env={"BFB_CKPT": str(tmp_path / "root_only.pth.tar")})


def test_neighbor_operation_sweeps():
    run_ranks("neighbor_sweeps", 4, timeout=400)


def test_neighbor_operation_sweeps_three_ranks():
    run_ranks("neighbor_sweeps", 3, timeout=400)


def test_associated_p_follows_random_weights():
    run_ranks("win_random_p", 4, timeout=300)


def test_local_step_warning_and_duplicated_layers():
    run_ranks("optimizer_warnings", 2, timeout=300)


def test_rank_that_leaves_is_detected():
    run_ranks("rank_exits_early", 3, timeout=120)


def test_stall_warning_names_missing_rank():
    out = run_ranks("stall_warning", 2, timeout=120)
    assert "late.tensor" in out[0][1] and "missing ranks: 1" in out[0][1]


def test_window_guard_words_detect_a_write_past_the_tensor():
    run_ranks("win_guard", 2, timeout=300)


def test_runtime_counters_and_their_prometheus_view():
    run_ranks("runtime_stats", 3, timeout=300)
