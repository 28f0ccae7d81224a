"""One rank of the multi-GPU context tests; launched by torch.distributed.run.

Every rank builds the same group-wide inputs deterministically, so each can
check its own outputs against the CPU oracle without exchanging anything.
"""

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ep_xpress_b200 import Config, Context, get_nccl_comm_handle  # noqa: E402
from ep_xpress_b200.ops import scale_rows  # noqa: E402
from ep_xpress_b200.utils import routing, workloads  # noqa: E402


def bits(t):
    return t.detach().cpu().contiguous().view(torch.int16)


def group_inputs(case, world, tokens, hidden, topk, iteration):
    xs, ids, ws = [], [], []
    for rank in range(world):
        if case == "uniform":
            n = max(tokens - 2 * rank, 0) if iteration % 2 else tokens
            i, w = workloads.uniform_routing(n, world * 4, topk, seed=iteration, rank=rank)
        else:
            i, w, _ = workloads.replay_case(case, rank=rank, world_size=world, tokens=tokens, topk=topk,
                                            iteration=iteration)
        xs.append(workloads.marker_payload(i.shape[0], hidden, rank=rank, iteration=iteration))
        ids.append(i)
        ws.append(w)
    return xs, ids, ws


def expected(xs, ids, ws, emap, world, topk, hidden, factors):
    plan = routing.plan_routes(ids, ws, emap, world, topk)
    rows = routing.dispatch_oracle(xs, plan)
    partials = [routing.scale_expert_oracle(rows[r], plan.received[r].local_ids, plan.received[r].weights, factors[r])
                for r in range(world)]
    return plan, rows, routing.combine_oracle(partials, plan, hidden)


def check_batch(batch, plan, rows, rank):
    valid = int(batch.valid_count.item())
    routes = plan.received[rank]
    assert valid == routes.rows, (valid, routes.rows)
    assert torch.equal(bits(batch.hidden[:valid]), bits(rows[rank]))
    assert torch.equal(batch.local_ids[:valid].cpu(), routes.local_ids)
    assert torch.equal(batch.weights[:valid].cpu(), routes.weights)
    assert torch.equal(batch.handle.inverse_map[:valid].cpu(), routes.inverse)
    assert (batch.local_ids[valid:] == -1).all() and (batch.weights[valid:] == 0).all()
    assert (batch.hidden[valid:].view(torch.int16) == 0).all()


def run_replay(ep, rank, world, args):
    hidden, topk, tokens = args.hidden, 4, args.tokens
    emap = workloads.contiguous_expert_map(world * 4, world)
    factors = [(r * 4 + torch.arange(4, dtype=torch.float32) + 1) / 8 for r in range(world)]
    my_factors = factors[rank].cuda()
    for case in workloads.REPLAY_CASES + ("uniform",):
        for iteration in range(2):
            xs, ids, ws = group_inputs(case, world, tokens, hidden, topk, iteration)
            plan, rows, want = expected(xs, ids, ws, emap, world, topk, hidden, factors)
            x, i, w = xs[rank].cuda(), ids[rank].cuda(), ws[rank].cuda()
            if iteration % 2:
                i = i.to(torch.int32)
            batch = ep.dispatch_async(x, i, w, tag=[case, iteration]).wait()
            check_batch(batch, plan, rows, rank)
            if iteration % 2:
                partial = scale_rows(ep, batch, my_factors)                       # zero-copy plane
            else:
                partial = scale_rows(ep, batch, my_factors, out=torch.zeros_like(batch.hidden))  # caller tensor
            out = ep.combine_async(partial, batch.handle, tag=[case, iteration]).wait()
            assert torch.equal(bits(out), bits(want[rank])), f"{case} iteration {iteration}: combine differs"
            try:
                ep.combine_async(partial, batch.handle)
            except ValueError as error:
                assert "already been consumed" in str(error)
            else:
                raise AssertionError("a handle was combined twice")
    ep.check()


def run_reverse_handles(ep, rank, world, args):
    """Two dispatches outstanding, combined in reverse (rank-consistent) order."""
    hidden, topk, tokens = args.hidden, 4, args.tokens
    emap = workloads.contiguous_expert_map(world * 4, world)
    factors = [torch.ones(4) for _ in range(world)]
    stream = torch.cuda.current_stream()
    held = []
    for iteration in range(2):
        xs, ids, ws = group_inputs("uniform", world, tokens, hidden, topk, iteration)
        plan, rows, want = expected(xs, ids, ws, emap, world, topk, hidden, factors)
        batch = ep.dispatch_on_stream(xs[rank].cuda(), ids[rank].cuda(), ws[rank].cuda(), stream=stream)
        check_batch(batch, plan, rows, rank)
        held.append((batch, want))
    for batch, want in reversed(held):
        out = ep.combine_on_stream(scale_rows(ep, batch), batch.handle, stream=stream)
        assert torch.equal(bits(out), bits(want[rank]))
    try:
        for iteration in range(3):
            xs, ids, ws = group_inputs("uniform", world, tokens, hidden, topk, iteration)
            ep.dispatch_on_stream(xs[rank].cuda(), ids[rank].cuda(), ws[rank].cuda(), stream=stream)
    except RuntimeError as error:
        assert "slots" in str(error)
    else:
        raise AssertionError("a third outstanding handle must be rejected with slots=2")


def run_graph(ep, rank, world, args):
    """Decode workspace captured once, replayed with changing routes, eager prefill interleaved."""
    hidden, topk, tokens = args.hidden, 4, args.tokens
    emap = workloads.contiguous_expert_map(world * 4, world)
    factors = [torch.ones(4) for _ in range(world)]
    ep.enable_cuda_graph()
    workspace = ep.create_workspace(world * tokens, tokens)
    stream = torch.cuda.Stream()
    static = [torch.zeros((tokens, hidden), dtype=torch.bfloat16, device="cuda"),
              torch.zeros((tokens, topk), dtype=torch.int64, device="cuda"),
              torch.zeros((tokens, topk), dtype=torch.float32, device="cuda")]

    def layer():
        batch = ep.dispatch_on_stream(*static, stream=stream, workspace=workspace)
        partial = scale_rows(ep, batch, stream=stream)
        return ep.combine_on_stream(partial, batch.handle, stream=stream), batch

    def load(iteration):
        xs, ids, ws = group_inputs("mixed" if iteration % 3 else "padding", world, tokens, hidden, topk, iteration)
        for dst, src in zip(static, (xs[rank], ids[rank], ws[rank])):
            dst.copy_(src)
        return expected(xs, ids, ws, emap, world, topk, hidden, factors)

    with torch.cuda.stream(stream):
        load(0)
        layer()                                   # warm the workspace eagerly
    stream.synchronize()
    try:
        with torch.cuda.stream(stream):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                layer()
    except RuntimeError as error:
        assert "prepare_graph_capture" in str(error)
    else:
        raise AssertionError("capture without prepare_graph_capture must be rejected")
    torch.cuda.synchronize()
    ep.prepare_graph_capture()
    ep.prepare_decode_profile(stage="combine")      # fixed counters the captured combine keeps writing
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        out, batch = layer()
    for iteration in range(1, args.replays + 1):
        with torch.cuda.stream(stream):
            plan, rows, want = load(iteration)
            ep.prepare_graph_replay(stream)
            graph.replay()
        stream.synchronize()
        check_batch(batch, plan, rows, rank)
        assert torch.equal(bits(out), bits(want[rank])), f"replay {iteration} differs"
        if iteration % 4 == 0:                    # an eager operation between replays
            xs, ids, ws = group_inputs("uniform", world, tokens, hidden, topk, 100 + iteration)
            _, _, eager_want = expected(xs, ids, ws, emap, world, topk, hidden, factors)
            eager = ep.dispatch_async(xs[rank].cuda(), ids[rank].cuda(), ws[rank].cuda()).wait()
            result = ep.combine_async(scale_rows(ep, eager), eager.handle).wait()
            assert torch.equal(bits(result), bits(eager_want[rank]))
    decode = ep.stop_decode_profile()
    assert decode["stage"] == "combine" and decode["phases"]["start"]["first_ns"] == 0
    assert decode["phases"]["reduced"]["last_ns"] > 0
    ep.check()


def run_errors(ep, rank, world, args):
    """A capacity that is too small poisons the group within the timeout; the GPU stays usable."""
    hidden, topk, tokens = args.hidden, 4, args.tokens
    xs, ids, ws = group_inputs("hotspot", world, tokens, hidden, topk, 0)
    batch = ep.dispatch_async(xs[rank].cuda(), ids[rank].cuda(), ws[rank].cuda(), recv_capacity=1).wait()
    try:
        ep.check()
    except RuntimeError as error:
        text = str(error)
        assert ("capacity" in text) or ("peer aborted" in text) or ("timed out" in text), text
    else:
        raise AssertionError("an undersized capacity must surface at check()")
    try:
        ep.dispatch_async(xs[rank].cuda(), ids[rank].cuda(), ws[rank].cuda())
    except RuntimeError as error:
        assert "failed state" in str(error)
    else:
        raise AssertionError("a poisoned context must refuse new work")
    assert torch.ones(2, device="cuda").sum().item() == 2
    del batch


def run_profile(ep, rank, world, args):
    """Bounded operation profile: per-CTA phase stamps, dropped operations, single readback."""
    hidden, topk, tokens = args.hidden, 4, args.tokens
    stream = torch.cuda.current_stream()
    try:
        ep.read_combine_profile()
    except RuntimeError as error:
        assert "no completed" in str(error)
    ep.start_combine_profile(max_operations=4)
    try:
        ep.start_combine_profile()
    except RuntimeError as error:
        assert "stop the current" in str(error)
    ep.set_combine_profile_label("warm")
    for iteration in range(3):                       # 6 operations, room for 4
        xs, ids, ws = group_inputs("uniform", world, tokens, hidden, topk, iteration)
        batch = ep.dispatch_on_stream(xs[rank].cuda(), ids[rank].cuda(), ws[rank].cuda(), stream=stream)
        ep.combine_on_stream(scale_rows(ep, batch), batch.handle, stream=stream)
    report = ep.stop_combine_profile()
    assert report is ep.read_combine_profile()
    assert len(report["operations"]) == 4 and report["dropped_operations"] == 2
    kinds = [op["kind"] for op in report["operations"]]
    assert kinds == ["dispatch", "combine", "dispatch", "combine"]
    for op in report["operations"]:
        assert op["label"] == "warm" and op["elapsed_ns"] > 0 and op["ctas"] >= 1
        names = list(op["phases"])
        assert names[0] == "start" and op["phases"]["start"]["first_ns"] == 0
        lasts = [op["phases"][n]["last_ns"] for n in names]
        assert lasts == sorted(lasts), (op["kind"], lasts)      # phases are reached in order
    stats = ep.stats()
    assert stats["status"] == 0 and stats["dispatch_epoch"] == 3 and stats["combine_epoch"] == 3
    try:
        ep.start_combine_profile(max_operations=1 << 30)
    except ValueError as error:
        assert "64 MiB budget" in str(error)
    ep.check()


CASES = {"profile": run_profile, "replay": run_replay, "reverse": run_reverse_handles, "graph": run_graph, "errors": run_errors}


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--case", choices=sorted(CASES), required=True)
    parser.add_argument("--hidden", type=int, default=256)
    parser.add_argument("--tokens", type=int, default=24)
    parser.add_argument("--replays", type=int, default=12)
    args = parser.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    comm = get_nccl_comm_handle(dist.group.WORLD)
    cfg = Config(hidden_size=args.hidden, topk=4, max_tokens_per_rank=args.tokens,
                 timeout_seconds=2.0 if args.case == "errors" else 10.0)
    emap = workloads.contiguous_expert_map(world * 4, world)
    ep = Context(nccl_comm=comm, expert_to_rank=emap, config=cfg)
    try:
        CASES[args.case](ep, rank, world, args)
    finally:
        ep.close()
    # the borrowed communicator is still usable after close
    probe = torch.ones(1, device="cuda")
    dist.all_reduce(probe)
    assert probe.item() == world
    dist.destroy_process_group()
    print(f"rank {rank}: {args.case} ok", flush=True)


if __name__ == "__main__":
    main()
