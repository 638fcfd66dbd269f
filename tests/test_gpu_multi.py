"""The multi-process cases of tests/_worker.py on real GPUs (one process per GPU, CUDA-IPC
peer memory over NVLink).  Skipped when the box has fewer GPUs than ranks."""
import os

import pytest
import torch

from conftest import run_ranks

pytestmark = pytest.mark.gpu

NVLS_OFF = {"NCCL_NVLS_ENABLE": "0"}


def _need(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.parametrize("case", ["collectives", "neighbor_ops", "windows", "optimizers", "gpu_fused_optimizers",
                                  "gpu_fast_path", "gpu_pair_gossip", "gpu_fused_wrap_then_broadcast",
                                  "gpu_fused_dst_weights_and_hierarchical", "neighbor_sweeps", "win_random_p",
                                  "gpu_registered_tensors", "win_guard"])
def test_two_gpus(case):
    _need(2)
    run_ranks(case, 2, gpu=True, env=NVLS_OFF, timeout=600)


@pytest.mark.parametrize("case", ["collectives", "neighbor_ops", "windows", "gpu_fused_optimizers",
                                  "gpu_fast_path", "gpu_pair_gossip", "gpu_fused_wrap_then_broadcast", "neighbor_sweeps",
                                  "gpu_registered_tensors"])
def test_four_gpus(case):
    _need(4)
    run_ranks(case, 4, gpu=True, env=NVLS_OFF, timeout=600)


def test_hierarchical_four_gpus():
    _need(4)
    run_ranks("hierarchical", 4, gpu=True, env=dict(NVLS_OFF, BLUEFOG_NODES_PER_MACHINE="2"), timeout=600)


def test_fused_hierarchical_and_destination_weights_four_gpus():
    _need(4)
    run_ranks("gpu_fused_dst_weights_and_hierarchical", 4, gpu=True, env=dict(NVLS_OFF, BLUEFOG_NODES_PER_MACHINE="2"),
              timeout=600)


@pytest.mark.parametrize("case", ["neighbor_ops", "collectives", "windows", "gpu_fused_optimizers",
                                  "gpu_fused_wrap_then_broadcast"])
def test_eight_gpus(case):
    _need(8)
    run_ranks(case, 8, gpu=True, env=NVLS_OFF, timeout=600)


def test_pattern_mismatch_times_out_with_an_error_on_gpus():
    """A rank waits for a peer that does not publish to it: the device wait gives up after the
    (shortened) limit and the operation raises instead of hanging."""
    _need(2)
    run_ranks("gpu_wait_timeout", 2, gpu=True, env=dict(NVLS_OFF, BLUEFOG_B200_WAIT_TIMEOUT_MS="300"), timeout=300)


def test_timeline_has_device_spans_on_gpus(tmp_path):
    _need(2)
    prefix = str(tmp_path / "tl_")
    run_ranks("gpu_timeline", 2, gpu=True, env=dict(NVLS_OFF, BLUEFOG_TIMELINE=prefix), timeout=300)
