"""Failure propagation of the host-staged and the multi-node transport within a bound, on CPU ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29502 -m benchmarks.failure_replay

A tag that differs between ranks and a token that selects an expert twice must both be
reported on EVERY rank before ``Config.timeout_seconds`` passes, and poison the context
(the reference's benchmarks/failure_replay.py:1-66, host_ce cases). The multi-node transport
(``internode_transport="gin"``) is replayed with an invalid route and an undersized capacity on
one rank. Runs over gloo: no GPU.
"""

from __future__ import annotations

import os
import sys
import time

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ep_xpress_b200 import Config, Context  # noqa: E402
from ep_xpress_b200.comm import GroupControlPlane  # noqa: E402
from ep_xpress_b200.utils import workloads  # noqa: E402


def attempt(case, rank, world):
    cfg = Config(hidden_size=64, topk=2, max_tokens_per_rank=16, transport="host_ce", timeout_seconds=5.0)
    emap = workloads.round_robin_expert_map(world * 2, world)
    ep = Context(GroupControlPlane(), emap, cfg)
    ids, w = workloads.uniform_routing(16, world * 2, 2, seed=1, rank=rank)
    x = workloads.gaussian_payload(16, 64, seed=1, rank=rank)
    tag = "layer"
    if case == "tag":
        tag = ("layer", rank)
    elif rank == world - 1:
        ids[0, 1] = ids[0, 0]
    begin = time.monotonic()
    try:
        ep.dispatch_async(x, ids, w, tag=tag).wait()
    except (RuntimeError, ValueError) as error:
        elapsed = time.monotonic() - begin
        assert elapsed < cfg.timeout_seconds, elapsed
        try:
            ep.dispatch_async(x, ids, w)
        except RuntimeError as again:
            assert "failed state" in str(again)
        ep.close()
        return f"{case}: {type(error).__name__} after {elapsed * 1e3:.1f} ms"
    raise AssertionError(f"{case}: the fault was not reported on rank {rank}")


def attempt_multinode(case, rank, world):
    cfg = Config(hidden_size=64, topk=2, max_tokens_per_rank=16, transport="host_sm", internode_transport="gin",
                 timeout_seconds=5.0)
    emap = workloads.round_robin_expert_map(world * 2, world)
    ep = Context(GroupControlPlane(), emap, cfg)
    ids, w = workloads.uniform_routing(16, world * 2, 2, seed=1, rank=rank)
    x = workloads.gaussian_payload(16, 64, seed=1, rank=rank)
    capacity = None
    if case == "invalid_route" and rank == world - 1:
        ids[0, 1] = ids[0, 0]
    if case == "capacity":
        capacity = 1
    begin = time.monotonic()
    try:
        ep.dispatch_async(x, ids, w, recv_capacity=capacity).wait()
    except RuntimeError as error:
        elapsed = time.monotonic() - begin
        assert elapsed < cfg.timeout_seconds, elapsed
        try:
            ep.dispatch_async(x, ids, w)
        except RuntimeError as again:
            assert "failed state" in str(again)
        ep.close()
        return f"multinode {case}: {type(error).__name__} after {elapsed * 1e3:.1f} ms"
    raise AssertionError(f"multinode {case}: the fault was not reported on rank {rank}")


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lines = [attempt(case, rank, world) for case in ("tag", "invalid_route")]
    lines += [attempt_multinode(case, rank, world) for case in ("invalid_route", "capacity")]
    dist.barrier()
    if rank == 0:
        print("failure replay ok: " + "; ".join(lines))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
