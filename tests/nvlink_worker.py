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
    """Several decode buckets captured once each, replayed in turn with routes that change at every
    replay; one bucket leaves a rank without tokens; eager operations run between replays; a
    bounded sample ring records every operation (scenario of the reference's
    tests/test_host_sm_graph_cuda.py:87-122,180-188)."""
    hidden, topk, tokens = args.hidden, 4, args.tokens
    emap = workloads.contiguous_expert_map(world * 4, world)
    factors = [torch.ones(4) for _ in range(world)]
    ep.enable_cuda_graph()
    stream = torch.cuda.Stream()
    # Bucket b gives rank r `sizes[b][r]` tokens; the last bucket empties the highest rank.
    sizes = [[tokens] * world, [max(tokens // 2 - r, 1) for r in range(world)], [1] * world,
             [tokens - 1 if r + 1 < world else 0 for r in range(world)]]
    fused = bool(ep.config.decode_max_tokens)

    def inputs(bucket, iteration):
        xs, ids, ws = [], [], []
        case = "mixed" if iteration % 3 else "padding"
        for r in range(world):
            n = sizes[bucket][r]
            i, w, _ = workloads.replay_case(case, rank=r, world_size=world, tokens=n, topk=topk, iteration=iteration)
            xs.append(workloads.marker_payload(n, hidden, rank=r, iteration=iteration))
            ids.append(i[:n])
            ws.append(w[:n])
        return xs, ids, ws

    buckets = []
    for b, per_rank in enumerate(sizes):
        n = per_rank[rank]
        workspace = ep.create_workspace(sum(per_rank), n, fused_combine=fused)
        static = [torch.zeros((n, hidden), dtype=torch.bfloat16, device="cuda"),
                  torch.zeros((n, topk), dtype=torch.int64, device="cuda"),
                  torch.zeros((n, topk), dtype=torch.float32, device="cuda")]
        buckets.append({"workspace": workspace, "static": static})

    def layer(bucket):
        batch = ep.dispatch_on_stream(*bucket["static"], stream=stream, workspace=bucket["workspace"],
                                      fused_combine=fused)
        partial = scale_rows(ep, batch, stream=stream)
        return ep.combine_on_stream(partial, batch.handle, stream=stream), batch

    def load(b, iteration):
        xs, ids, ws = inputs(b, iteration)
        for dst, src in zip(buckets[b]["static"], (xs[rank], ids[rank], ws[rank])):
            dst.copy_(src)
        return expected(xs, ids, ws, emap, world, topk, hidden, factors)

    with torch.cuda.stream(stream):
        for b in range(len(buckets)):
            load(b, 0)
            layer(buckets[b])                     # warm every workspace eagerly
    stream.synchronize()
    try:
        with torch.cuda.stream(stream):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                layer(buckets[0])
    except RuntimeError as error:
        assert "prepare_graph_capture" in str(error)
    else:
        raise AssertionError("capture without prepare_graph_capture must be rejected")
    torch.cuda.synchronize()
    ep.prepare_decode_profile(max_samples_per_channel=64, stage="layer")
    ep.prepare_graph_capture()
    for bucket in buckets:
        bucket["graph"] = torch.cuda.CUDAGraph()
        with torch.cuda.graph(bucket["graph"], stream=stream):
            bucket["out"], bucket["batch"] = layer(bucket)
    ep.start_decode_profile()
    operations = 0
    for iteration in range(1, args.replays + 1):
        b = (iteration * 7 + iteration // 5) % len(buckets)          # bucket switches in an irregular order
        bucket = buckets[b]
        with torch.cuda.stream(stream):
            plan, rows, want = load(b, iteration)
            ep.prepare_graph_replay(stream)
            bucket["graph"].replay()
        operations += 1
        if iteration % args.check_every == 0 or iteration <= 40 or iteration == args.replays:
            stream.synchronize()
            check_batch(bucket["batch"], plan, rows, rank)
            assert torch.equal(bits(bucket["out"]), bits(want[rank])), f"replay {iteration} (bucket {b}) differs"
        if iteration % 16 == 0:                   # an eager operation between replays
            xs, ids, ws = group_inputs("uniform", world, tokens, hidden, topk, 100 + iteration)
            _, _, eager_want = expected(xs, ids, ws, emap, world, topk, hidden, factors)
            eager = ep.dispatch_async(xs[rank].cuda(), ids[rank].cuda(), ws[rank].cuda()).wait()
            result = ep.combine_async(scale_rows(ep, eager), eager.handle).wait()
            assert torch.equal(bits(result), bits(eager_want[rank]))
            operations += 1
    decode = ep.stop_decode_profile()
    assert decode["stage"] == "layer" and set(decode["stages"]) == {"dispatch", "combine"}
    for name, stage in decode["stages"].items():
        # The ring is bounded: 64 samples are kept, every later operation is counted as dropped.
        assert stage["samples"] == min(operations, 64), (name, stage["samples"], operations)
        assert stage["dropped_samples"] == max(operations - 64, 0), (name, stage["dropped_samples"], operations)
        assert all(0 < ns < 5_000_000_000 for ns in stage["elapsed_ns"])
        assert stage["begin_ns"] == sorted(stage["begin_ns"])
    ep.check()


def _layer_once(ep, x, ids, ws, *, stream=None, direct=True, factors=None, out=None):
    if direct:
        batch = ep.dispatch_on_stream(x, ids, ws, stream=stream)
        partial = scale_rows(ep, batch, factors, stream=stream, out=out)
        return ep.combine_on_stream(partial, batch.handle, stream=stream), batch
    batch = ep.dispatch_async(x, ids, ws, stream=stream).wait(stream)
    partial = scale_rows(ep, batch, factors, stream=stream, out=out)
    return ep.combine_async(partial, batch.handle, stream=stream).wait(stream), batch


def run_streams(ep, rank, world, args):
    """Ticket API and direct-stream API interleaved on different streams, with consumers of the
    results on yet another stream (scenario of the reference's tests/test_host_sm_stream_cuda.py:69-75)."""
    hidden, topk, tokens = args.hidden, 4, args.tokens
    emap = workloads.contiguous_expert_map(world * 4, world)
    factors = [torch.ones(4) for _ in range(world)]
    streams = [torch.cuda.Stream() for _ in range(3)]
    consumer = torch.cuda.Stream()
    checks = []
    for iteration in range(12):
        xs, ids, ws = group_inputs("uniform", world, tokens, hidden, topk, iteration)
        _, _, want = expected(xs, ids, ws, emap, world, topk, hidden, factors)
        stream = streams[iteration % 3]
        with torch.cuda.stream(stream):
            x, i, w = xs[rank].cuda(non_blocking=True), ids[rank].cuda(non_blocking=True), ws[rank].cuda(non_blocking=True)
            out, _ = _layer_once(ep, x, i, w, stream=stream, direct=iteration % 2 == 0)
        consumer.wait_stream(stream)
        with torch.cuda.stream(consumer):                 # a consumer on another stream reads the result
            checks.append((out.clone(), want[rank]))
            out.record_stream(consumer)
    torch.cuda.synchronize()
    for got, want in checks:
        assert torch.equal(bits(got), bits(want))
    ep.check()


def run_stagger(ep, rank, world, args):
    """Ranks that arrive late and readers that lag: before each of 32 back-to-back layers one
    rank (a different one every time) stalls its stream, so its peers' rows wait in its planes and
    its own rows arrive after everybody else's (scenario of the reference's
    tests/test_host_sm_mailbox_reclaim_cuda.py:100-107 and test_host_sm_ready_prefetch_cuda.py:117-143)."""
    hidden, topk, tokens = args.hidden, 4, args.tokens
    emap = workloads.contiguous_expert_map(world * 4, world)
    factors = [torch.ones(4) for _ in range(world)]
    workspace = ep.create_workspace(world * tokens, tokens)
    stream = torch.cuda.current_stream()
    results = []
    for iteration in range(32):
        if iteration % 2:
            routes = [workloads.uniform_routing(tokens, world * 4, topk, seed=iteration, rank=r) for r in range(world)]
            ids, ws = [i for i, _ in routes], [w for _, w in routes]
            xs = [workloads.marker_payload(tokens, hidden, rank=r, iteration=iteration) for r in range(world)]
        else:
            xs, ids, ws = group_inputs("mixed", world, tokens, hidden, topk, iteration)
        _, _, want = expected(xs, ids, ws, emap, world, topk, hidden, factors)
        x, i, w = xs[rank].cuda(), ids[rank].cuda(), ws[rank].cuda()
        if iteration % world == rank:
            torch.cuda._sleep(3_000_000)                  # about 1.5 ms of a 2 GHz clock
        batch = ep.dispatch_on_stream(x, i, w, stream=stream, workspace=workspace)
        partial = scale_rows(ep, batch, stream=stream)
        if (iteration + 1) % world == rank:
            torch.cuda._sleep(3_000_000)                  # this rank pushes late, its reducers wait
        out = ep.combine_on_stream(partial, batch.handle, stream=stream)
        results.append((out.clone(), want[rank]))
    torch.cuda.synchronize()
    for index, (got, want) in enumerate(results):
        assert torch.equal(bits(got), bits(want)), f"layer {index} differs"
    ep.check()


def run_headline(ep, rank, world, args):
    """The benchmarked shape (hidden 7168, 4096 tokens per rank, 256 experts, top-8), checked bit
    for bit on this rank: received rows against the senders' inputs, output against the
    rank-order FP32 formula."""
    hidden, topk, tokens, experts = args.hidden, 8, args.tokens, 256
    emap = workloads.contiguous_expert_map(experts, world)
    owner = torch.tensor(emap)
    for seed in range(2):
        routes = [workloads.uniform_routing(tokens, experts, topk, seed=seed, rank=r, weights="sigmoid")
                  for r in range(world)]
        xs = [workloads.gaussian_payload(tokens, hidden, seed=seed, rank=r) for r in range(world)]
        x, ids, w = xs[rank].cuda(), routes[rank][0].cuda(), routes[rank][1].cuda()
        batch = ep.dispatch_on_stream(x, ids, w)
        partial = scale_rows(ep, batch)
        out = ep.combine_on_stream(partial, batch.handle)
        torch.cuda.synchronize()
        valid = int(batch.valid_count.item())
        want_rows = sum(int((owner[i] == rank).any(dim=1).sum()) for i, _ in routes)
        assert valid == want_rows, (valid, want_rows)
        inverse = batch.handle.inverse_map[:valid].cpu()
        everything = torch.stack(xs)                                   # [world, tokens, hidden]
        assert torch.equal(bits(batch.hidden[:valid]), bits(everything[inverse[:, 0], inverse[:, 1]]))
        assert (inverse[1:, 0] * tokens + inverse[1:, 1] > inverse[:-1, 0] * tokens + inverse[:-1, 1]).all()
        want = routing.identity_layer_oracle(xs[rank], routes[rank][0], routes[rank][1], emap, rank, world)
        assert torch.equal(bits(out), bits(want)), f"seed {seed}: combine output differs"
    ep.check()


def run_host_ce(comm, rank, world, args):
    """The host-staged oracle transport on CUDA tensors over the borrowed NCCL communicator: its
    combine runs on the native add_partial / finish_combine kernels."""
    hidden, topk, tokens, experts = 128, 4, 29, world * 4
    emap = workloads.round_robin_expert_map(experts, world)
    for rounding in ("two_step", "single"):
        cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=32, transport="host_ce",
                     chunk_bytes=hidden * 2 * 8, timeout_seconds=30.0, combine_rounding=rounding)
        with Context(nccl_comm=comm, expert_to_rank=emap, config=cfg) as ep:
            xs, ids, ws = group_inputs("uniform", world, tokens, hidden, topk, 1)
            ids = [workloads.uniform_routing(i.shape[0], experts, topk, seed=2, rank=r)[0] for r, i in enumerate(ids)]
            plan = routing.plan_routes(ids, ws, emap, world, topk)
            rows = routing.dispatch_oracle(xs, plan)
            batch = ep.dispatch_async(xs[rank].cuda(), ids[rank].cuda(), ws[rank].cuda(), tag="oracle").wait()
            assert batch.valid_count == plan.received[rank].rows and batch.hidden.is_cuda
            assert torch.equal(bits(batch.hidden), bits(rows[rank]))
            partials = [routing.scale_expert_oracle(rows[r], plan.received[r].local_ids, plan.received[r].weights)
                        for r in range(world)]
            out = ep.combine_async(partials[rank].cuda(), batch.handle, tag="oracle").wait()
            want = routing.combine_oracle(partials, plan, hidden, rounding)
            assert out.is_cuda and torch.equal(bits(out), bits(want[rank])), rounding


def run_topk(comm, rank, world, args):
    """top-k 3 and 33 with a placement that is neither contiguous nor balanced (one rank owns no
    expert when there are at least three) - scenario of the reference's
    tests/test_dispatch_route_tiles_cuda.py:105-114."""
    hidden, tokens, experts = 192, 37, 40
    owners = [(e * 7 + 3) % world for e in range(experts)]
    if world >= 3:
        owners = [o if o != 1 else 0 for o in owners]                  # rank 1 owns nothing
    for topk in (3, 33):
        cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=tokens, timeout_seconds=10.0)
        with Context(nccl_comm=comm, expert_to_rank=owners, config=cfg) as ep:
            for iteration in range(3):
                routes = [workloads.uniform_routing(tokens - r, experts, topk, seed=iteration, rank=r) for r in range(world)]
                ids, ws = [i for i, _ in routes], [w for _, w in routes]
                if iteration == 1:
                    ids = [i.to(torch.int32) for i in ids]
                xs = [workloads.marker_payload(tokens - r, hidden, rank=r, iteration=iteration) for r in range(world)]
                per_rank = [owners.count(r) for r in range(world)]
                factors = [torch.arange(1, max(n, 1) + 1, dtype=torch.float32) / 4 for n in per_rank]
                plan, rows, want = expected(xs, [i.to(torch.int64) for i in ids], ws, owners, world, topk, hidden, factors)
                batch = ep.dispatch_async(xs[rank].cuda(), ids[rank].cuda(), ws[rank].cuda(), tag=iteration).wait()
                check_batch(batch, plan, rows, rank)
                out = ep.combine_async(scale_rows(ep, batch, factors[rank].cuda()), batch.handle, tag=iteration).wait()
                assert torch.equal(bits(out), bits(want[rank])), f"topk {topk} iteration {iteration}: combine differs"
            ep.check()


def run_subgroup(rank, world, args):
    """An EP group over a NON-contiguous subgroup ([0, 2] of four ranks); on one member the handle
    object is dropped and garbage-collected and then looked up again - that must not communicate
    (the other member does not call anything) - and the subgroup's communicator still works
    after the context is closed (scenario of the reference's tests/test_nccl_comm_cuda.py:46-87)."""
    import gc
    members = [0, 2]
    group = dist.new_group(members)                     # collective over ALL ranks
    if rank in members:
        comm = get_nccl_comm_handle(group)              # collective over the subgroup (warms it up)
        assert (comm.rank, comm.world_size) == (members.index(rank), 2)
        pointer = comm.get()
        if rank == 0:
            del comm
            gc.collect()
        torch.cuda.synchronize()
        comm = get_nccl_comm_handle(group)              # rank 0: a fresh handle object, no collective
        assert comm.get() == pointer
        hidden, topk, tokens = 128, 2, 16
        emap = workloads.round_robin_expert_map(4, 2)
        cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=tokens, timeout_seconds=10.0)
        me = members.index(rank)
        with Context(nccl_comm=comm, expert_to_rank=emap, config=cfg) as ep:
            routes = [workloads.uniform_routing(tokens, 4, topk, seed=9, rank=r) for r in range(2)]
            xs = [workloads.marker_payload(tokens, hidden, rank=r, iteration=0) for r in range(2)]
            ids, ws = [i for i, _ in routes], [w for _, w in routes]
            plan, rows, want = expected(xs, ids, ws, emap, 2, topk, hidden, [torch.ones(2)] * 2)
            batch = ep.dispatch_async(xs[me].cuda(), ids[me].cuda(), ws[me].cuda()).wait()
            check_batch(batch, plan, rows, me)
            out = ep.combine_async(scale_rows(ep, batch), batch.handle).wait()
            assert torch.equal(bits(out), bits(want[me]))
            try:
                Context(nccl_comm=comm, expert_to_rank=emap, config=cfg, device=torch.device("cuda", (rank + 1) % world))
            except ValueError as error:
                assert "same CUDA device" in str(error)
            else:
                raise AssertionError("a context on another device than its communicator must be rejected")
        probe = torch.ones(1, device="cuda")
        dist.all_reduce(probe, group=group)             # the borrowed communicator survives close()
        assert probe.item() == 2
    dist.barrier()


def run_multinode(comm, rank, world, args):
    """The multi-node context on GPUs: the ranks of ONE box are labelled as two nodes, records move
    with grouped NCCL point-to-point transfers on the borrowed communicator, and every plane is
    compared with the oracle (the CPU-rank test of the same path: tests/test_multinode_gloo.py)."""
    hidden, topk, tokens, experts = 256, 3, 21, world * 3
    emap = [(e * 7) % world for e in range(experts)]
    os.environ["EPX_NODE_ID"] = f"node{rank * 2 // world}"          # two node labels on one box
    for rounding in ("auto", "two_step"):
        cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=32, transport="host_sm",
                     internode_transport="gin", combine_rounding=rounding, max_pending_operations=2)
        ep = Context(comm, emap, cfg)
        assert type(ep).__name__ == "MultiNodeContext" and ep.device.type == "cuda"
        assert ep.transport_info["nodes"] == 2 and rank in ep.transport_info["local_ranks"]
        handles = []
        for seed in (1, 2):
            routes = [workloads.uniform_routing(max(tokens - 4 * r, 0), experts, topk, seed=seed, rank=r) for r in range(world)]
            ids, ws = [i for i, _ in routes], [w for _, w in routes]
            xs = [workloads.gaussian_payload(i.shape[0], hidden, seed=seed, rank=r) for r, i in enumerate(ids)]
            plan = routing.plan_routes(ids, ws, emap, world, topk)
            batch = ep.dispatch_async(xs[rank].cuda(), (ids[rank] if seed == 1 else ids[rank].to(torch.int32)).cuda(),
                                      ws[rank].cuda(), tag=("layer", seed)).wait()
            want = plan.received[rank]
            valid = int(batch.valid_count.item())
            assert batch.hidden.is_cuda and valid == want.rows
            assert torch.equal(bits(batch.hidden[:valid]), bits(routing.dispatch_oracle(xs, plan)[rank]))
            assert torch.equal(batch.local_ids[:valid].cpu(), want.local_ids)
            assert torch.equal(batch.handle.inverse_map[:valid].cpu(), want.inverse)
            assert (batch.local_ids[valid:] == -1).all() and (batch.hidden[valid:] == 0).all()
            partial = routing.scale_expert_oracle(batch.hidden[:valid].cpu(), batch.local_ids[:valid].cpu(),
                                                  batch.weights[:valid].cpu())
            padded = torch.zeros_like(batch.hidden)
            padded[:valid] = partial.cuda()
            handles.append((batch.handle, padded, xs, plan, seed))
        for handle, padded, xs, plan, seed in reversed(handles):
            out = ep.combine_async(padded, handle, tag=("layer", seed)).wait()
            rows = routing.dispatch_oracle(xs, plan)
            partials = [routing.scale_expert_oracle(rows[r], plan.received[r].local_ids, plan.received[r].weights)
                        for r in range(world)]
            want_out = routing.combine_oracle(partials, plan, hidden, "two_step" if rounding == "two_step" else "single")
            assert out.is_cuda and torch.equal(bits(out), bits(want_out[rank])), (rounding, seed)
        ep.close()


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
    """Bounded operation profile: per-CTA phase stamps and counters, dropped operations, single readback."""
    from ep_xpress_b200.utils.profile import check_invariants
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
        check_invariants(op, row_bytes=hidden * 2)               # disjoint phases sum to elapsed, bytes = rows x row
        assert op["protocol"] in ("bulk", "mailbox") and op["polls"] >= 0
        assert op["rows"] > 0 or (op["kind"] == "combine" and world == 1)     # a lone rank pushes nothing
        if world > 1:
            assert op["first_publish_ns"] is not None and op["first_receive_ns"] is not None
    stats = ep.stats()
    assert stats["status"] == 0 and stats["dispatch_epoch"] == 3 and stats["combine_epoch"] == 3
    try:
        ep.start_combine_profile(max_operations=1 << 30)
    except ValueError as error:
        assert "64 MiB budget" in str(error)
    ep.check()


CASES = {"streams": run_streams, "stagger": run_stagger, "headline": run_headline, "profile": run_profile, "replay": run_replay, "reverse": run_reverse_handles, "graph": run_graph, "errors": run_errors}


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--case", choices=sorted(CASES) + ["hostce", "multinode", "topk", "subgroup"], required=True)
    parser.add_argument("--hidden", type=int, default=256)
    parser.add_argument("--tokens", type=int, default=24)
    parser.add_argument("--replays", type=int, default=1000)
    parser.add_argument("--check-every", type=int, default=1)
    parser.add_argument("--decode-max-tokens", type=int, default=0)
    args = parser.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    comm = get_nccl_comm_handle(dist.group.WORLD)
    if args.case in ("topk", "subgroup", "multinode"):
        if args.case == "topk":
            run_topk(comm, rank, world, args)
        elif args.case == "multinode":
            run_multinode(comm, rank, world, args)
        else:
            run_subgroup(rank, world, args)
        dist.destroy_process_group()
        print(f"rank {rank}: {args.case} ok", flush=True)
        return
    if args.case == "hostce":
        run_host_ce(comm, rank, world, args)
        dist.destroy_process_group()
        print(f"rank {rank}: hostce ok", flush=True)
        return
    if args.case == "headline":
        cfg = Config(hidden_size=args.hidden, topk=8, max_tokens_per_rank=args.tokens, timeout_seconds=20.0)
        ep = Context(nccl_comm=comm, expert_to_rank=workloads.contiguous_expert_map(256, world), config=cfg)
        try:
            run_headline(ep, rank, world, args)
        finally:
            ep.close()
        dist.destroy_process_group()
        print(f"rank {rank}: headline ok", flush=True)
        return
    cfg = Config(hidden_size=args.hidden, topk=4, max_tokens_per_rank=args.tokens,
                 decode_max_tokens=args.decode_max_tokens, slots=2,
                 workspace_pool_bytes=(8 << 20) + 6 * Config(hidden_size=args.hidden, topk=4,
                                                             max_tokens_per_rank=args.tokens).nvlink_slot_bytes(world),
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
