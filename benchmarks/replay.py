"""Correctness replay of the device transport against the CPU oracle, under torchrun.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        --master-port 29501 -m benchmarks.replay --iterations 4 [--expect-error capacity] [--delay-rank 1]

Seven route cases (mixed, empty, local, hotspot, all_empty, padding, all_padding) with
position-marker payloads, checked bit for bit: received rows, local ids, weights, inverse
map, padding, and the rank-order BF16 combine. ``--expect-error`` injects one fault on the
host side of the API (invalid id, duplicate expert, NaN weight, capacity 0, consumed handle)
and checks that it surfaces as the documented error without hanging any rank;
``--delay-rank`` makes one rank enter every operation late; ``--profile-combine`` runs every
operation with the profiling kernels and checks the report's invariants (every CTA reaches the
last phase, disjoint phases sum to the CTA's elapsed time, bytes = rows x row size, rows
stored = rows the route plan sends; the checks of the reference's harness,
benchmarks/replay.py:185-268). Behavioural re-creation of that harness (benchmarks/replay.py:19-473).
"""

from __future__ import annotations

import argparse
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ep_xpress_b200 import Config, Context, get_nccl_comm_handle  # noqa: E402
from ep_xpress_b200.ops import scale_rows  # noqa: E402
from ep_xpress_b200.utils import routing, workloads  # noqa: E402

ERRORS = ("none", "invalid_id", "duplicate", "nan_weight", "capacity", "consumed")


def bits(t):
    return t.detach().cpu().contiguous().view(torch.int16)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--iterations", type=int, default=3)
    parser.add_argument("--tokens", type=int, default=24)
    parser.add_argument("--hidden", type=int, default=256)
    parser.add_argument("--expect-error", choices=ERRORS, default="none")
    parser.add_argument("--delay-rank", type=int, default=-1)
    parser.add_argument("--profile-combine", action="store_true")
    args = parser.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    topk, per_rank = 4, 4
    emap = workloads.contiguous_expert_map(world * per_rank, world)
    cfg = Config(hidden_size=args.hidden, topk=topk, max_tokens_per_rank=args.tokens,
                 timeout_seconds=3.0 if args.expect_error != "none" else 20.0)
    ep = Context(get_nccl_comm_handle(dist.group.WORLD), emap, cfg)
    factors = [(r * per_rank + torch.arange(per_rank, dtype=torch.float32) + 1) / 8 for r in range(world)]
    mine = factors[rank].cuda()
    profiled = []
    try:
        for case in workloads.REPLAY_CASES:
            for iteration in range(args.iterations):
                if args.profile_combine:
                    ep.start_combine_profile(max_operations=4)
                    ep.set_combine_profile_label(f"{case}/{iteration}")
                xs, ids, ws = [], [], []
                for r in range(world):
                    i, w, _ = workloads.replay_case(case, rank=r, world_size=world, tokens=args.tokens, topk=topk,
                                                    experts_per_rank=per_rank, iteration=iteration)
                    xs.append(workloads.marker_payload(i.shape[0], args.hidden, rank=r, iteration=iteration))
                    ids.append(i)
                    ws.append(w)
                plan = routing.plan_routes(ids, ws, emap, world, topk)
                rows = routing.dispatch_oracle(xs, plan)
                partials = [routing.scale_expert_oracle(rows[r], plan.received[r].local_ids,
                                                        plan.received[r].weights, factors[r]) for r in range(world)]
                want = routing.combine_oracle(partials, plan, args.hidden)
                if rank == args.delay_rank:
                    time.sleep(0.02)
                batch = ep.dispatch_async(xs[rank].cuda(), ids[rank].cuda(), ws[rank].cuda(),
                                          tag=[case, iteration]).wait()
                valid = int(batch.valid_count.item())
                routes = plan.received[rank]
                assert valid == routes.rows
                assert torch.equal(bits(batch.hidden[:valid]), bits(rows[rank]))
                assert torch.equal(batch.local_ids[:valid].cpu(), routes.local_ids)
                assert torch.equal(batch.weights[:valid].cpu(), routes.weights)
                assert torch.equal(batch.handle.inverse_map[:valid].cpu(), routes.inverse)
                assert (batch.local_ids[valid:] == -1).all() and (batch.hidden[valid:].view(torch.int16) == 0).all()
                out = ep.combine_async(scale_rows(ep, batch, mine), batch.handle, tag=[case, iteration]).wait()
                assert torch.equal(bits(out), bits(want[rank])), (case, iteration)
                if args.profile_combine:
                    report = ep.stop_combine_profile()
                    profiled.append(check_profile(report, plan, rank, world, args.hidden, f"{case}/{iteration}"))
        ep.check()
        if args.expect_error != "none":
            inject(ep, args, rank, world, topk, per_rank)
    finally:
        ep.close()
    probe = torch.ones(1, device="cuda")
    dist.all_reduce(probe)
    dist.destroy_process_group()
    if rank == 0 and profiled:
        print(f"profile ok: {len(profiled)} dispatch/combine pairs, dispatch p50 "
              f"{sorted(p[0] for p in profiled)[len(profiled) // 2]} ns, combine p50 "
              f"{sorted(p[1] for p in profiled)[len(profiled) // 2]} ns on rank 0")
    if rank == 0:
        print(f"replay ok: {len(workloads.REPLAY_CASES)} cases x {args.iterations} iterations on {world} ranks"
              + (f", error '{args.expect_error}' surfaced as documented" if args.expect_error != "none" else ""))


def check_profile(report, plan, rank, world, hidden, label):
    """Invariants of one profiled dispatch/combine pair; returns their elapsed times (ns)."""
    from ep_xpress_b200.utils.profile import check_invariants
    assert report["dropped_operations"] == 0 and [op["kind"] for op in report["operations"]] == ["dispatch", "combine"]
    dispatch, combine = report["operations"]
    assert dispatch["label"] == combine["label"] == label
    for entry in (dispatch, combine):
        check_invariants(entry, row_bytes=hidden * 2)
    sent = int((plan.dest_rows[rank] >= 0).sum())                       # rows this rank's tokens go to
    owed = plan.received[rank].rows - int((plan.received[rank].source_rank == rank).sum())
    assert dispatch["rows"] == sent, (dispatch["rows"], sent)
    assert combine["rows"] == owed, (combine["rows"], owed)            # rows pushed back to other ranks
    if world > 1 and sent:
        assert dispatch["first_publish_ns"] is not None and dispatch["first_receive_ns"] is not None
    return dispatch["elapsed_ns"], combine["elapsed_ns"]


def inject(ep, args, rank, world, topk, per_rank):
    ids, w, _ = workloads.replay_case("mixed", rank=rank, world_size=world, tokens=args.tokens, topk=topk,
                                      experts_per_rank=per_rank)
    x = workloads.marker_payload(ids.shape[0], args.hidden, rank=rank)
    kwargs = {}
    if args.expect_error == "consumed":
        batch = ep.dispatch_async(x.cuda(), ids.cuda(), w.cuda()).wait()
        partial = scale_rows(ep, batch)
        ep.combine_async(partial, batch.handle).wait()
        try:
            ep.combine_async(partial, batch.handle)
        except ValueError as error:
            assert "already been consumed" in str(error)
            return
        raise AssertionError("a consumed handle was accepted")
    if rank == 0:
        if args.expect_error == "invalid_id":
            ids[0, 0] = world * per_rank + 3
        elif args.expect_error == "duplicate":
            ids[0, 1] = ids[0, 0]
        elif args.expect_error == "nan_weight":
            w[0, 0] = float("nan")
    if args.expect_error == "capacity":
        kwargs["recv_capacity"] = 0
    ep.dispatch_async(x.cuda(), ids.cuda(), w.cuda(), **kwargs).wait()
    try:
        ep.check()
    except RuntimeError as error:
        text = str(error)
        assert any(word in text for word in ("invalid route", "capacity", "peer aborted", "timed out")), text
    else:
        raise AssertionError("the injected error did not surface at check()")
    assert torch.ones(2, device="cuda").sum().item() == 2      # the GPU is still usable


if __name__ == "__main__":
    main()
