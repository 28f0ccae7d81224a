"""host_ce end to end on CPU ranks over gloo: routing, chunked ring exchange, rank-order combine,
tag mismatch and invalid-route propagation (the reference's failure_replay cases)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ep_xpress_b200 import Config, Context
from ep_xpress_b200.comm import GroupControlPlane
from ep_xpress_b200.utils import routing, workloads


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        hidden, topk, tokens, experts = 64, 2, 37, world * 2
        cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=64, transport="host_ce",
                     chunk_bytes=hidden * 2 * 8, slots=2, timeout_seconds=20.0,
                     combine_rounding="single" if case == "single" else "two_step")
        emap = workloads.round_robin_expert_map(experts, world)
        ep = Context(GroupControlPlane(), emap, cfg, shared_directory=tmp)
        xs, ids, ws = [], [], []
        for r in range(world):
            n = tokens - 5 * r
            i, w = workloads.uniform_routing(n, experts, topk, seed=3, rank=r)
            if r == 0:
                i[1, :] = -1
                w[1, :] = float("nan")
            xs.append(workloads.gaussian_payload(n, hidden, seed=3, rank=r))
            ids.append(i)
            ws.append(w)
        if case == "invalid" and rank == 1:
            ids[1] = ids[1].clone()
            ids[1][0, 1] = ids[1][0, 0]
        if case == "tag":
            with pytest.raises(RuntimeError, match="mismatch"):
                ep.dispatch_async(xs[rank], ids[rank], ws[rank], tag=("a", rank)).wait()
            with pytest.raises(RuntimeError, match="failed state"):
                ep.dispatch_async(xs[rank], ids[rank], ws[rank])
            ep.close()
            dist.barrier()
            return
        if case == "invalid":
            with pytest.raises(ValueError, match="same expert twice"):
                ep.dispatch_async(xs[rank], ids[rank], ws[rank]).wait()
            ep.close()
            dist.barrier()
            return
        plan = routing.plan_routes(ids, ws, emap, world, topk)
        rows = routing.dispatch_oracle(xs, plan)
        ticket = ep.dispatch_async(xs[rank], ids[rank], ws[rank], tag="layer0")
        batch = ticket.wait()
        assert ticket.done and ticket.metrics["chunks_sent"] >= 1
        assert batch.valid_count == plan.received[rank].rows
        assert torch.equal(batch.hidden.view(torch.int16), rows[rank].view(torch.int16))
        assert torch.equal(batch.local_ids, plan.received[rank].local_ids)
        assert torch.equal(batch.weights, plan.received[rank].weights)
        partials = [routing.scale_expert_oracle(rows[r], plan.received[r].local_ids, plan.received[r].weights)
                    for r in range(world)]
        out = ep.combine_async(partials[rank], batch.handle, tag="layer0").wait()
        want = routing.combine_oracle(partials, plan, hidden, cfg.combine_rounding)
        assert torch.equal(out.view(torch.int16), want[rank].view(torch.int16))
        with pytest.raises(ValueError, match="already been consumed"):
            ep.combine_async(partials[rank], batch.handle)
        with pytest.raises(ValueError, match="only supported by host_sm"):
            ep.dispatch_async(xs[rank], ids[rank], ws[rank], recv_capacity=4)
        ep.check()
        ep.close()
        dist.barrier()                      # nobody tears the group down while a peer still uses it
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,case", [(2, "two_step"), (3, "single"), (2, "tag"), (2, "invalid")])
def test_host_ce(world, case, tmp_path):
    mp.spawn(_worker, args=(world, _free_port(), case, str(tmp_path)), nprocs=world, join=True)
