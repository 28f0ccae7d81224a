"""The NVLink context as a one-rank group: the whole public path (borrowed NCCL handle, heap,
kernels, tickets, graphs, profile) on a single GPU."""

import pytest

from conftest import gpu_count
from test_nvlink_multigpu import launch

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(gpu_count() < 1, reason="needs a CUDA device")]


@pytest.mark.parametrize("case", ["replay", "graph", "profile", "reverse"])
def test_one_rank_group(case):
    launch(case, 1)
