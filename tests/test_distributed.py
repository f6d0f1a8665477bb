"""Multi-process CPU tests (gloo): process topology, distributed transforms / norm / loss / channel-parallel MLP against
their serial counterparts (forward and gradients, uneven splits), flexible checkpoints across layouts.
Pattern of the reference's tests/distributed/tests_fft.py:94-244: split -> op -> uneven gather -> compare."""

import os
import socket
import subprocess
import sys
import tempfile

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(case, sizes, world, cuda=False):
    port = _free_port()
    procs = []
    tmp = tempfile.mkdtemp()
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="1", MK_TMP=tmp)
        if cuda:
            # one GPU per rank; in-switch reductions off so that a failing rank cannot disturb its peers' GPUs
            env.update(MK_DEVICE="cuda", NCCL_NVLS_ENABLE="0")
        else:
            env.update(CUDA_VISIBLE_DEVICES="")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "dist_worker.py"), case] + [str(s) for s in sizes],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "WORKER_OK" in out, f"rank {r} failed:\n{out[-3000:]}"


def test_compute_group_ranks_layout():
    from makani_b200.utils.comm import compute_group_ranks
    g = compute_group_ranks(16, dict(h=2, w=2, fin=2, fout=1))
    assert g["model"] == [list(range(0, 8)), list(range(8, 16))]
    assert g["data"][0] == [0, 8]
    assert g["fin"][0] == [0, 1] and g["w"][0] == [0, 2] and g["h"][0] == [0, 4]
    assert g["spatial"][0] == [0, 2, 4, 6] and g["matmul"][0] == [0, 1]


def test_split_shapes():
    from makani_b200.parallel.helpers import compute_split_shapes
    assert compute_split_shapes(721, 4) == [181, 181, 181, 178]
    assert compute_split_shapes(721, 8) == [91] * 7 + [84]
    assert compute_split_shapes(241, 2) == [121, 120]
    assert compute_split_shapes(241, 8) == [31] * 7 + [24]
    assert compute_split_shapes(8, 8) == [1] * 8


@pytest.mark.parametrize("sizes,world", [((2, 2, 1, 1), 4), ((1, 1, 2, 1), 4)])
def test_topology(sizes, world):
    _launch("topology", sizes, world)


@pytest.mark.parametrize("sizes", [(2, 1, 1, 1), (1, 2, 1, 1), (2, 2, 1, 1)])
def test_distributed_sht(sizes):
    _launch("sht", sizes, sizes[0] * sizes[1])


def test_distributed_fft():
    _launch("fft", (2, 2, 1, 1), 4)


def test_distributed_norm_and_loss():
    _launch("norm_and_loss", (2, 2, 1, 1), 4)


@pytest.mark.parametrize("sizes", [(1, 1, 2, 1), (1, 1, 1, 2), (1, 1, 2, 2)])
def test_channel_parallel_mlp(sizes):
    _launch("matmul", sizes, sizes[2] * sizes[3])


@pytest.mark.parametrize("sizes", [(2, 1, 1, 1), (2, 2, 1, 1)])
def test_spatially_parallel_sfno_matches_serial(sizes):
    _launch("sfno_and_checkpoint", sizes, sizes[0] * sizes[1])


@pytest.mark.parametrize("sizes", [(2, 1, 1, 1), (1, 2, 1, 1), (2, 2, 1, 1), (3, 1, 1, 1)])
def test_fused_distributed_spectral_conv(sizes):
    _launch("fused_spectral", sizes, sizes[0] * sizes[1])


@pytest.mark.parametrize("sizes", [(1, 1, 2, 1), (1, 1, 1, 2), (1, 1, 2, 2)])
def test_fused_channel_parallel_matmul_algebra(sizes):
    _launch("fused_matmul", sizes, sizes[2] * sizes[3])


@pytest.mark.parametrize("sizes", [(1, 1, 2, 1), (1, 1, 2, 2)])
def test_distributed_patch_embed(sizes):
    _launch("patch_embed", sizes, sizes[2] * sizes[3])


@pytest.mark.parametrize("world", [2, 3])
def test_gradient_reduction_hooks_in_a_plain_loop(world):
    """`init_gradient_reduction_hooks` (the upstream entry point for user loops) on 2 and 3 data-parallel ranks."""
    _launch("reduction_hooks", (1, 1, 1, 1), world)


@pytest.mark.parametrize("sizes", [(1, 1, 1, 2), (1, 1, 2, 1), (1, 1, 2, 2)])
def test_channel_parallel_attention_matches_serial(sizes):
    _launch("attention", sizes, sizes[2] * sizes[3])
