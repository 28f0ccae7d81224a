"""End-to-end tests of the NVLink context on real GPUs, one process per GPU over NCCL
(the reference's tier of spawned multi-GPU tests, e.g. tests/test_host_sm_graph_cuda.py)."""

import os
import socket
import subprocess
import sys

import pytest

from conftest import gpu_count


WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "nvlink_worker.py")


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch(case, ranks, *extra, timeout=420):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), WORKER, "--case", case, *extra]
    result = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert result.returncode == 0, result.stdout[-3000:] + "\n" + result.stderr[-3000:]


def ranks_available():
    return [n for n in (2, 4, 8) if n <= gpu_count()]


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(gpu_count() < 2, reason="needs at least two CUDA devices")
@pytest.mark.parametrize("ranks", ranks_available() or [2])
def test_replay_cases(ranks):
    launch("replay", ranks)


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(gpu_count() < 2, reason="needs at least two CUDA devices")
def test_reverse_order_handles():
    launch("reverse", min(gpu_count(), 4))


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(gpu_count() < 2, reason="needs at least two CUDA devices")
def test_cuda_graph_replay_with_changing_routes():
    """1000 replays over four captured buckets (one leaves a rank empty); the first 40 replays and
    every fourth one after them are checked against the oracle."""
    launch("graph", min(gpu_count(), 4), "--replays", "1000", "--check-every", "4", timeout=900)


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(gpu_count() < 2, reason="needs at least two CUDA devices")
def test_cuda_graph_replay_at_decode_size_with_fused_combine():
    launch("graph", min(gpu_count(), 4), "--hidden", "7168", "--tokens", "128", "--replays", "300",
           "--check-every", "10", "--decode-max-tokens", "128", timeout=900)


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(gpu_count() < 2, reason="needs at least two CUDA devices")
def test_ticket_and_direct_calls_across_streams():
    launch("streams", min(gpu_count(), 4))


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(gpu_count() < 2, reason="needs at least two CUDA devices")
def test_staggered_ranks_and_lagging_readers():
    launch("stagger", min(gpu_count(), 4))


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(gpu_count() < 2, reason="needs at least two CUDA devices")
def test_benchmarked_shape_is_bit_exact():
    launch("headline", min(gpu_count(), 8), "--hidden", "7168", "--tokens", "4096", timeout=900)


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(gpu_count() < 2, reason="needs at least two CUDA devices")
def test_undersized_capacity_poisons_the_group_without_hanging():
    launch("errors", 2)


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(gpu_count() < 2, reason="needs at least two CUDA devices")
def test_operation_profile():
    launch("profile", 2)


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(gpu_count() < 2, reason="needs at least two CUDA devices")
def test_host_staged_transport_on_cuda_tensors():
    launch("hostce", 2)


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(gpu_count() < 2, reason="needs at least two CUDA devices")
def test_topk_3_and_33_with_a_scattered_expert_map():
    launch("topk", min(gpu_count(), 4))


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(gpu_count() < 3, reason="needs at least three CUDA devices")
def test_noncontiguous_subgroup_and_handle_reacquisition():
    launch("subgroup", min(gpu_count(), 4))


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(gpu_count() < 2, reason="needs at least two CUDA devices")
def test_multinode_context_over_nccl_point_to_point():
    launch("multinode", min(gpu_count(), 4))
