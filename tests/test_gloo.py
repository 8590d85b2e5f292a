"""CPU/gloo multi-process tests of the operator surface: correctness against torch.distributed,
autograd, validation, subgroups and FakeTensor shape propagation. No GPU needed.
Modelled on the reference's test/distributed/{correctness,validation,subgroup}.py, run over the
CPU backend this library adds."""

import pytest

from _dist import run_ranks


def test_config1_round_trip_ws2():
    run_ranks(2, "_gloo_workers", "round_trip_config1")


def test_round_trip_ws3():
    run_ranks(3, "_gloo_workers", "round_trip_config1")


@pytest.mark.parametrize("world", [1, 2, 4])
def test_even_and_dtypes(world):
    run_ranks(world, "_gloo_workers", "even_and_dtypes")


def test_autograd_ws2():
    run_ranks(2, "_gloo_workers", "autograd_paths")


def test_autograd_ws3():
    run_ranks(3, "_gloo_workers", "autograd_paths")


def test_validation_ws2():
    run_ranks(2, "_gloo_workers", "validation")


def test_subgroups_ws4():
    run_ranks(4, "_gloo_workers", "subgroups")


def test_fake_tensor_ws2():
    run_ranks(2, "_gloo_workers", "fake_tensor")
