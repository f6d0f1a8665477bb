"""Multi-GPU tests (one process per GPU, NCCL + peer memory): the fused compute+communication kernels against their
serial counterparts.  Skipped when the machine has fewer GPUs than the case needs."""

import pytest
import torch

from test_distributed import _launch

pytestmark = pytest.mark.gpu


def _need(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.parametrize("sizes", [(1, 2, 1, 1), (2, 1, 1, 1)])
def test_fused_distributed_spectral_conv_2gpu(sizes):
    _need(2)
    _launch("fused_spectral", sizes, 2, cuda=True)


def test_fused_distributed_spectral_conv_4gpu():
    _need(4)
    _launch("fused_spectral", (2, 2, 1, 1), 4, cuda=True)


@pytest.mark.parametrize("sizes,world", [((2, 1, 1, 1), 2), ((2, 2, 1, 1), 4)])
def test_peer_memory_instance_norm(sizes, world):
    _need(world)
    _launch("peer_instance_norm", sizes, world, cuda=True)


@pytest.mark.parametrize("sizes,world", [((1, 1, 2, 1), 2), ((1, 1, 1, 2), 2), ((1, 1, 2, 2), 4)])
def test_fused_channel_parallel_matmul(sizes, world):
    _need(world)
    _launch("fused_matmul", sizes, world, cuda=True)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_allreduce_matches_nccl(world):
    _need(world)
    _launch("peer_allreduce", (1, 1, 1, 1), world, cuda=True)


@pytest.mark.parametrize("sizes,world", [((2, 1, 1, 1), 2), ((2, 2, 1, 1), 4), ((2, 1, 1, 1), 4), ((4, 2, 1, 1), 8)])
def test_peer_shared_parameter_sums(sizes, world):
    _need(world)
    _launch("peer_shared_sums", sizes, world, cuda=True)


@pytest.mark.parametrize("sizes,world", [((2, 1, 1, 1), 2), ((1, 2, 1, 1), 2), ((2, 2, 1, 1), 4)])
def test_fused_chains_repeat_bitwise(sizes, world):
    _need(world)
    _launch("fused_repeat", sizes, world, cuda=True)
