"""Multi-GPU tests: one process per GPU over NCCL, at min(n_gpu, 8) ranks and also at 3 ranks when
there are at least 3 GPUs (odd world sizes). Modelled on the reference's test/distributed/*.py:
bit-exact correctness against torch.distributed, uniform validation, the ordering control with its
in-process negative control, CUDA-graph replay with epoch equality, sync/async coexistence, the
window-reuse race, subgroups, and a host-made peer failure that the bounded waits must report."""

import os

import pytest
import torch

from _dist import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def world_sizes():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    env = os.environ.get("FU_TEST_NPROC")
    if env:
        return [int(env)]
    sizes = [min(n, 8)] if n >= 2 else []
    if n >= 3 and 3 not in sizes:
        sizes.append(3)
    return sizes or [2]


@pytest.fixture(autouse=True)
def _plain_peer_access(monkeypatch):
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")


@pytest.mark.parametrize("world", world_sizes())
def test_correctness(world):
    run_ranks(world, "_gpu_workers", "correctness", backend="nccl", timeout=600)


@pytest.mark.parametrize("world", world_sizes()[:1])
def test_validation_is_uniform(world):
    run_ranks(world, "_gpu_workers", "validation_uniform", backend="nccl", timeout=300)


@pytest.mark.parametrize("world", world_sizes()[:1])
def test_ordering_control(world):
    run_ranks(world, "_gpu_workers", "ordering_control", backend="nccl", timeout=300)


@pytest.mark.parametrize("world", world_sizes()[:1])
def test_graph_replay(world):
    run_ranks(world, "_gpu_workers", "graph_replay", backend="nccl", timeout=300)


@pytest.mark.parametrize("world", world_sizes()[:1])
def test_sync_async_coexist(world):
    run_ranks(world, "_gpu_workers", "sync_async_coexist", backend="nccl", timeout=600)


@pytest.mark.parametrize("world", world_sizes())
def test_output_pool(world):
    run_ranks(world, "_gpu_workers", "output_pool", backend="nccl", timeout=300)


@pytest.mark.parametrize("world", world_sizes()[:1])
def test_window_reuse_race(world):
    run_ranks(world, "_gpu_workers", "window_reuse_race", backend="nccl", timeout=300)


@pytest.mark.parametrize("world", world_sizes()[:1])
def test_async_input_may_be_overwritten(world):
    run_ranks(world, "_gpu_workers", "async_input_may_be_overwritten", backend="nccl", timeout=300)


@pytest.mark.parametrize("world", world_sizes())
def test_copy_engine_transport(world):
    run_ranks(world, "_gpu_workers", "copy_engine_transport", backend="nccl", timeout=600)


@pytest.mark.parametrize("world", world_sizes()[:1])
def test_pooled_result_read_on_a_side_stream(world):
    run_ranks(world, "_gpu_workers", "pooled_result_read_on_a_side_stream", backend="nccl", timeout=300)


def test_subgroups():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if n < 4:
        pytest.skip("needs an even world of at least 4")
    run_ranks(4, "_gpu_workers", "subgroups_gpu", backend="nccl", timeout=300)


@pytest.mark.parametrize("world", world_sizes()[:1])
def test_peer_timeout_is_reported(world):
    run_ranks(world, "_gpu_workers", "peer_timeout_is_reported", backend="nccl", timeout=300)


@pytest.mark.parametrize("world", world_sizes())
def test_sp_attention_block(world):
    run_ranks(world, "_gpu_workers", "sp_attention_block", backend="nccl", timeout=300)


@pytest.mark.parametrize("world", world_sizes()[:1])
def test_fused_block_beside_an_async_exchange(world):
    run_ranks(world, "_gpu_workers", "fused_block_beside_an_async_exchange", backend="nccl", timeout=300)


@pytest.mark.parametrize("world", world_sizes())
def test_fp8_exchange_fused(world):
    run_ranks(world, "_gpu_workers", "fp8_exchange_fused", backend="nccl", timeout=300)


@pytest.mark.parametrize("world", world_sizes()[:1])
def test_dit_stack(world):
    if world not in (2, 4, 8):
        pytest.skip("even world sizes")
    run_ranks(world, "_gpu_workers", "dit_stack", backend="nccl", timeout=300)


@pytest.mark.parametrize("world", world_sizes()[:1])
def test_nvlink_probe_matches_nvml_oracle(world):
    run_ranks(world, "_gpu_workers", "nvlink_probe_matches_nvml_oracle", backend="nccl", timeout=200)
