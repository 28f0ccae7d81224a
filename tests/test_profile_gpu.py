"""Profiling specialisations of the transport kernels on one GPU (a group emulated inside single
launches): every CTA's disjoint phases sum to its elapsed time, bytes are rows times the row
size, the rows stored equal what the route plan sends, milestones lie inside the operation -
and the results stay bit-exact (invariants of the reference's
tests/test_host_sm_native_cuda.py:276-301)."""

import pytest
import torch

from conftest import gpu_count
from helpers import bits

from ep_xpress_b200 import Config, EmulatedGroup
from ep_xpress_b200.utils import profile, routing, workloads

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(gpu_count() < 1, reason="needs a CUDA device")]


@pytest.mark.parametrize("world,hidden,topk,tokens,protocol", [
    (4, 1024, 4, 96, "on"), (4, 1024, 4, 96, "off"), (2, 258, 2, 40, "on"), (1, 512, 2, 64, "on"), (3, 256, 3, 700, "on"),
])
def test_profile_invariants(world, hidden, topk, tokens, protocol, native):
    experts = world * 4
    cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=tokens, timeout_seconds=2.0,
                 combine_streaming=protocol)
    emap = workloads.round_robin_expert_map(experts, world)
    words = native.PROFILE_STAMPS
    with EmulatedGroup(world, emap, cfg) as group:
        dev = group.device
        slot = group.create_slot()
        routes = [workloads.uniform_routing(tokens - 3 * r, experts, topk, seed=4, rank=r) for r in range(world)]
        xs = [workloads.gaussian_payload(tokens - 3 * r, hidden, seed=4, rank=r) for r in range(world)]
        ids, ws = [i for i, _ in routes], [w for _, w in routes]
        plan = routing.plan_routes(ids, ws, emap, world, topk)
        ctas = 6
        records = {kind: torch.zeros((world, ctas, words), dtype=torch.int64, device=dev) for kind in ("dispatch", "combine")}
        with torch.cuda.device(dev):
            group.core.dispatch(slot, [x.to(dev) for x in xs], [i.to(dev) for i in ids], [w.to(dev) for w in ws],
                                [slot.capacity] * world, ctas=ctas, profile=records["dispatch"])
        batches = slot.views
        partials = [v.partial for v in batches]
        for rank, view in enumerate(batches):
            group.core.scale_rows(view.hidden, view.local_ids, view.weights, view.count, None, view.partial)
        outs = [torch.empty((x.shape[0], hidden), dtype=torch.bfloat16, device=dev) for x in xs]
        with torch.cuda.device(dev):
            group.core.combine(slot, partials, outs, ctas=ctas, profile=records["combine"])
        assert all(status[0] == 0 for status in group.status())
        rows = routing.dispatch_oracle(xs, plan)
        want_partials = [routing.scale_expert_oracle(rows[r], plan.received[r].local_ids, plan.received[r].weights)
                         for r in range(world)]
        want = routing.combine_oracle(want_partials, plan, hidden)
        for rank in range(world):
            assert torch.equal(bits(outs[rank]), bits(want[rank]))
            for kind in ("dispatch", "combine"):
                record = {"kind": kind, "operation": 1, "tag": None, "label": None, "tokens": xs[rank].shape[0],
                          "capacity": slot.capacity, "ctas": ctas}
                entry = profile.summarize(record, records[kind][rank].cpu())
                profile.check_invariants(entry, row_bytes=hidden * 2)
                if kind == "dispatch":
                    assert entry["rows"] == int((plan.dest_rows[rank] >= 0).sum())
                    assert entry["protocol"] == ("bulk" if hidden % 8 == 0 else "register")
                else:
                    routes_here = plan.received[rank]
                    assert entry["rows"] == routes_here.rows - int((routes_here.source_rank == rank).sum())
                    expected = "register" if hidden % 8 else ("bulk" if world == 1 or protocol == "off" else "mailbox")
                    assert entry["protocol"] == expected
                    assert entry["items"] > 0
