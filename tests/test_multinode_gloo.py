"""The multi-node transport on CPU ranks over gloo, two simulated nodes: record exchange,
(source rank, token) row order, zeroed non-local weights, single-rounding combine, tags,
bounded handles, and failures that reach every rank without a hang."""

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


def _inputs(world, experts, topk, hidden, tokens, seed):
    xs, ids, ws = [], [], []
    for r in range(world):
        n = max(tokens - 4 * r, 0)
        i, w = workloads.uniform_routing(n, experts, topk, seed=seed, rank=r)
        if r == 0 and n > 2:
            i[1, :] = -1
            w[1, :] = float("nan")                         # a padding token with ignored weights
            i[2, 0] = -1
        xs.append(workloads.gaussian_payload(n, hidden, seed=seed, rank=r))
        ids.append(i)
        ws.append(w)
    return xs, ids, ws


def _worker(rank, world, port, case):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), EPX_NODE_ID=f"node{rank // 2}")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        hidden, topk, tokens, experts = 64, 3, 21, world * 3
        rounding = "two_step" if case == "two_step" else "auto"
        cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=32, transport="host_sm",
                     internode_transport="gin", combine_rounding=rounding, max_pending_operations=2)
        emap = [(e * 7) % world for e in range(experts)]       # scattered placement
        ep = Context(GroupControlPlane(), emap, cfg)
        assert type(ep).__name__ == "MultiNodeContext"
        assert ep.transport_info["nodes"] == (world + 1) // 2 and rank in ep.transport_info["local_ranks"]
        if case in ("roundtrip", "two_step"):
            handles = []
            for seed in (1, 2):                                 # two handles outstanding, combined in reverse
                xs, ids, ws = _inputs(world, experts, topk, hidden, tokens, seed)
                plan = routing.plan_routes(ids, ws, emap, world, topk)
                batch = ep.dispatch_async(xs[rank], ids[rank] if seed == 1 else ids[rank].to(torch.int32), ws[rank],
                                          tag=("layer", seed)).wait()
                want = plan.received[rank]
                valid = int(batch.valid_count.item())
                assert valid == want.rows and batch.hidden.shape[0] == world * 32
                rows = routing.dispatch_oracle(xs, plan)[rank]
                assert torch.equal(batch.hidden[:valid].view(torch.int16), rows.view(torch.int16))
                assert torch.equal(batch.local_ids[:valid], want.local_ids)
                local = want.local_ids >= 0
                assert torch.equal(batch.weights[:valid], torch.where(local, want.weights, torch.zeros(())))
                assert (batch.local_ids[valid:] == -1).all() and (batch.weights[valid:] == 0).all()
                assert (batch.hidden[valid:] == 0).all() and (batch.handle.inverse_map[valid:] == -1).all()
                assert torch.equal(batch.handle.inverse_map[:valid], want.inverse)
                partial = routing.scale_expert_oracle(batch.hidden[:valid], batch.local_ids[:valid], batch.weights[:valid])
                padded = torch.zeros_like(batch.hidden)
                padded[:valid] = partial
                handles.append((batch.handle, padded, xs, plan, seed))
            with pytest.raises(RuntimeError, match="combine earlier handles"):
                ep.dispatch_async(xs[rank], ids[rank], ws[rank])
            for handle, padded, xs, plan, seed in reversed(handles):
                with pytest.raises(ValueError, match="tag differs"):
                    ep.combine_async(padded, handle, tag="other")
                out = ep.combine_async(padded, handle, tag=("layer", seed)).wait().clone()
                all_rows = routing.dispatch_oracle(xs, plan)
                partials = [routing.scale_expert_oracle(all_rows[r], plan.received[r].local_ids,
                                                        plan.received[r].weights) for r in range(world)]
                want_out = routing.combine_oracle(partials, plan, hidden, "two_step" if case == "two_step" else "single")
                assert torch.equal(out.view(torch.int16), want_out[rank].view(torch.int16))
                with pytest.raises(ValueError, match="unconsumed handle"):
                    ep.combine_async(padded, handle, tag=("layer", seed))
        elif case == "invalid":
            xs, ids, ws = _inputs(world, experts, topk, hidden, tokens, 3)
            if rank == 1:
                ids[1][0, 1] = ids[1][0, 0]                     # one rank routes a token to an expert twice
            with pytest.raises(RuntimeError, match=r"invalid route.*ranks \[1\]"):
                ep.dispatch_async(xs[rank], ids[rank], ws[rank])
            with pytest.raises(RuntimeError, match="failed state"):
                ep.dispatch_async(xs[rank], ids[rank], ws[rank])
        elif case == "capacity":
            xs, ids, ws = _inputs(world, experts, topk, hidden, tokens, 4)
            with pytest.raises(RuntimeError, match="capacity exceeded"):
                ep.dispatch_async(xs[rank], ids[rank], ws[rank], recv_capacity=3)
        with pytest.raises(NotImplementedError, match="cannot be captured"):
            ep.enable_cuda_graph()
        ep.close()
        dist.barrier()
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("world,case", [(4, "roundtrip"), (3, "two_step"), (4, "invalid"), (2, "capacity")])
def test_multinode_transport(world, case):
    mp.spawn(_worker, args=(world, _free_port(), case), nprocs=world, join=True)
