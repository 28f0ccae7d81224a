"""The multi-rank protocol on ONE GPU: all ranks inside single cooperative launches,
diffed bit for bit against the CPU oracle (technique of the reference's replay
harness, benchmarks/replay.py:67-125, with its seven route cases)."""

import pytest
import torch

from conftest import gpu_count
from helpers import bits, check_dispatch, expected_partials

from ep_xpress_b200 import Config, EmulatedGroup
from ep_xpress_b200.utils import routing, workloads

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(gpu_count() < 1, reason="needs a CUDA device")]


def run_round(group, slot, xs, ids, ws, expert_map, *, rounding="two_step", factors=None, capacities=None,
              direct_partial=True, ctas=None):
    world, cfg = group.world_size, group.config
    dev = group.device
    plan = routing.plan_routes(ids, ws, expert_map, world, cfg.topk)
    capacities = [slot.capacity] * world if capacities is None else capacities
    batches = group.dispatch(slot, [x.to(dev) for x in xs], [i.to(dev) for i in ids], [w.to(dev) for w in ws],
                             capacities, ctas=ctas)
    check_dispatch(batches, plan, xs, capacities, zero_padding=cfg.zero_padding)
    dev_factors = None if factors is None else [f.to(dev) for f in factors]
    partials = []
    for rank, batch in enumerate(batches):
        out = None if direct_partial else torch.zeros_like(batch.partial)
        partials.append(group.scale_rows(batch, None if dev_factors is None else dev_factors[rank], out))
    want_partials = expected_partials(plan, xs, factors)
    for rank in range(world):
        rows = plan.received[rank].rows
        assert torch.equal(bits(partials[rank][:rows]), bits(want_partials[rank])), f"rank {rank}: partial differs"
    outs = group.combine(slot, partials, [x.shape[0] for x in xs], ctas=ctas)
    want = routing.combine_oracle(want_partials, plan, cfg.hidden_size, rounding)
    for rank in range(world):
        assert torch.equal(bits(outs[rank]), bits(want[rank])), f"rank {rank}: combine output differs"
    assert all(status[0] == 0 for status in group.status())
    return plan


@pytest.mark.parametrize("world,hidden,topk,tokens", [
    (1, 64, 2, 17), (2, 256, 2, 64), (2, 258, 3, 5), (4, 264, 4, 33), (8, 2048, 8, 128), (3, 64, 4, 600),
])
def test_uniform_routes_bit_exact(world, hidden, topk, tokens):
    experts = world * 4
    cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=max(tokens, 8), timeout_seconds=2.0)
    emap = workloads.round_robin_expert_map(experts, world)
    with EmulatedGroup(world, emap, cfg) as group:
        slot = group.create_slot()
        for seed in range(3):
            xs, ids, ws = [], [], []
            for rank in range(world):
                n = tokens if seed != 1 else max(tokens - 3 * rank, 0)
                i, w = workloads.uniform_routing(n, experts, topk, seed=seed, rank=rank)
                xs.append(workloads.gaussian_payload(n, hidden, seed=seed, rank=rank))
                ids.append(i if seed % 2 == 0 else i.to(torch.int32))
                ws.append(w)
            factors = [torch.arange(1, 5, dtype=torch.float32) / 8 + rank for rank in range(world)]
            run_round(group, slot, xs, ids, ws, emap, factors=factors, direct_partial=(seed != 2))


@pytest.mark.parametrize("case", workloads.REPLAY_CASES)
def test_replay_cases(case):
    world, hidden, topk, tokens = 4, 128, 4, 19
    cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=tokens, timeout_seconds=2.0)
    emap = workloads.contiguous_expert_map(world * 4, world)
    with EmulatedGroup(world, emap, cfg) as group:
        slot = group.create_slot()
        for iteration in range(3):
            xs, ids, ws = [], [], []
            for rank in range(world):
                i, w, _ = workloads.replay_case(case, rank=rank, world_size=world, tokens=tokens, topk=topk,
                                                iteration=iteration)
                xs.append(workloads.marker_payload(i.shape[0], hidden, rank=rank, iteration=iteration))
                ids.append(i)
                ws.append(w)
            factors = [(rank * 4 + torch.arange(4, dtype=torch.float32) + 1) / 8 for rank in range(world)]
            run_round(group, slot, xs, ids, ws, emap, factors=factors)


def test_single_round_mode_and_noncontiguous_placement():
    world, hidden, topk, tokens = 4, 512, 3, 40
    cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=tokens, timeout_seconds=2.0,
                 combine_rounding="single")
    emap = [0, 2, 2, 0, 3, 0, 2, 3, 3]   # rank 1 owns no expert
    with EmulatedGroup(world, emap, cfg) as group:
        slot = group.create_slot()
        xs, ids, ws = [], [], []
        for rank in range(world):
            i, w = workloads.uniform_routing(tokens, len(emap), topk, seed=5, rank=rank)
            xs.append(workloads.gaussian_payload(tokens, hidden, seed=5, rank=rank))
            ids.append(i)
            ws.append(w)
        run_round(group, slot, xs, ids, ws, emap, rounding="single")


@pytest.mark.parametrize("world,topk", [(4, 3), (4, 33), (8, 33), (2, 33)])
def test_wide_topk_with_a_scattered_expert_map(world, topk):
    """top-k 3 and 33 (above the routed-from-registers width), a placement that is neither
    contiguous nor balanced, one rank without experts."""
    hidden, tokens, experts = 192, 37, 40
    owners = [(e * 7 + 3) % world for e in range(experts)]
    if world >= 3:
        owners = [o if o != 1 else 0 for o in owners]
    cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=tokens, timeout_seconds=2.0)
    with EmulatedGroup(world, owners, cfg) as group:
        slot = group.create_slot()
        for seed in range(3):
            routes = [workloads.uniform_routing(tokens - r, experts, topk, seed=seed, rank=r) for r in range(world)]
            xs = [workloads.marker_payload(tokens - r, hidden, rank=r, iteration=seed) for r in range(world)]
            ids = [i if seed != 1 else i.to(torch.int32) for i, _ in routes]
            run_round(group, slot, xs, ids, [w for _, w in routes], owners)


@pytest.mark.parametrize("rounding", ["two_step", "single"])
@pytest.mark.parametrize("hidden,tokens", [(7168, 300), (264, 41), (64, 1)])
def test_one_rank_group_streams_local_rows(hidden, tokens, rounding):
    """A group of one rank takes the streaming combine: tokens without any active expert come out
    as zeros, negative zeros come out as +0 like everywhere else, repeated operations keep the
    epoch in step, and a short partial is an error."""
    topk, experts = 4, 8
    cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=tokens, timeout_seconds=2.0,
                 combine_rounding=rounding)
    emap = [0] * experts
    with EmulatedGroup(1, emap, cfg) as group:
        slot = group.create_slot()
        for seed in range(3):
            ids, ws = workloads.uniform_routing(tokens, experts, topk, seed=seed, rank=0)
            x = workloads.gaussian_payload(tokens, hidden, seed=seed, rank=0)
            x[0, : hidden // 2] = -0.0
            if tokens > 2:
                ids[1] = -1                                     # a token that goes nowhere
                ws[2] = 0.0                                     # a token whose row is scaled to zero
            run_round(group, slot, [x], [ids], [ws], emap, rounding=rounding, direct_partial=(seed != 1))
        if tokens > 2:
            dev = group.device
            batch = group.dispatch(slot, [x.to(dev)], [ids.to(dev)], [ws.to(dev)])[0]
            short = group.scale_rows(batch)[: tokens - 2].clone()
            group.combine(slot, [short], [tokens])
            torch.cuda.synchronize()
            assert group.status()[0][0] != 0


def test_intermediate_rounding_is_observable():
    """remote-sum -> bf16 -> + local -> bf16 differs from a single rounding on chosen values."""
    world, hidden = 3, 64
    cfg = Config(hidden_size=hidden, topk=3, max_tokens_per_rank=1, timeout_seconds=2.0)
    emap = [0, 1, 2]
    with EmulatedGroup(world, emap, cfg) as group:
        slot = group.create_slot()
        dev = group.device
        ids = [torch.tensor([[0, 1, 2]]), torch.zeros((0, 3), dtype=torch.int64), torch.zeros((0, 3), dtype=torch.int64)]
        ws = [torch.ones((1, 3)), torch.zeros((0, 3)), torch.zeros((0, 3))]
        xs = [torch.ones((1, hidden), dtype=torch.bfloat16)] + [torch.zeros((0, hidden), dtype=torch.bfloat16)] * 2
        group.dispatch(slot, [x.to(dev) for x in xs], [i.to(dev) for i in ids], [w.to(dev) for w in ws])
        # rank 0 local = 1, rank 1 = 2**-9, rank 2 = 2**-9: the remote sum 2**-8 survives its own
        # rounding, then 1 + 2**-8 ties to even (1.0); a single rounding of 1 + 2**-8 gives the same,
        # so use values where the two-step result differs: remote 2**-8 + 2**-16.
        parts = [torch.full((3, hidden), 1.0), torch.full((3, hidden), 2.0 ** -8), torch.full((3, hidden), 2.0 ** -16)]
        parts = [p.to(torch.bfloat16).to(dev) for p in parts]
        outs = group.combine(slot, parts, [1, 0, 0])
        remote = (torch.tensor(2.0 ** -8) + torch.tensor(2.0 ** -16)).to(torch.bfloat16).to(torch.float32)
        want = (remote + 1.0).to(torch.bfloat16)
        single = (torch.tensor(1.0 + 2.0 ** -8 + 2.0 ** -16)).to(torch.bfloat16)
        assert want.item() != single.item()
        assert (outs[0].cpu() == want).all()


def test_capacity_exceeded_is_a_sticky_error_not_truncation():
    world, hidden, topk, tokens = 2, 64, 2, 16
    cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=tokens, timeout_seconds=0.5)
    emap = [0, 0, 1, 1]
    with EmulatedGroup(world, emap, cfg) as group:
        slot = group.create_slot()
        dev = group.device
        ids = [torch.tensor([[0, 2]] * tokens), torch.tensor([[1, 3]] * tokens)]
        ws = [torch.full((tokens, topk), 0.5)] * 2
        xs = [torch.ones((tokens, hidden), dtype=torch.bfloat16)] * 2
        batches = group.dispatch(slot, [x.to(dev) for x in xs], [i.to(dev) for i in ids], [w.to(dev) for w in ws],
                                 capacities=[4, 2 * tokens])
        statuses = group.status()
        assert statuses[0][0] == 2
        assert int(batches[0].valid_count.item()) == 0
        assert torch.ones(2, device=dev).sum().item() == 2   # the GPU is still usable


def test_invalid_routes_are_reported():
    world, hidden, topk, tokens = 2, 64, 2, 4
    cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=tokens, timeout_seconds=0.5)
    emap = [0, 1]
    for bad_ids, bad_w in (([[0, 0]], 0.5), ([[0, 7]], 0.5), ([[0, 1]], float("nan"))):
        with EmulatedGroup(world, emap, cfg) as group:
            slot = group.create_slot()
            dev = group.device
            ids = [torch.tensor(bad_ids * tokens), torch.tensor([[0, 1]] * tokens)]
            ws = [torch.full((tokens, topk), bad_w), torch.full((tokens, topk), 0.5)]
            xs = [torch.ones((tokens, hidden), dtype=torch.bfloat16)] * 2
            group.dispatch(slot, [x.to(dev) for x in xs], [i.to(dev) for i in ids], [w.to(dev) for w in ws])
            statuses = group.status()
            assert statuses[0][0] == 1
            assert statuses[1][0] in (0, 4)


@pytest.mark.parametrize("protocol", ["on", "off"])
@pytest.mark.parametrize("world,hidden,topk,tokens,ctas", [
    (2, 256, 2, 64, None),
    (4, 2048, 4, 700, None),      # several row segments per reduce item
    (8, 1024, 8, 300, 12),        # full fan-out, few CTAs per rank
    (3, 64, 4, 600, 5),           # tiny rows, more tokens than one route tile
    (4, 264, 4, 33, None),        # rows that are not 16-byte multiples: the register path runs instead
    (2, 8192, 2, 40, 7),          # rows larger than one mover / pusher stage: two pieces per row
])
def test_both_combine_protocols_match_the_oracle(world, hidden, topk, tokens, ctas, protocol):
    """Mailbox (push and reduce side by side, one arrival word per row) and sequential (push,
    signal, wait, reduce): both bit-exact, on uneven batches and skewed routes."""
    experts = world * 4
    cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=tokens, timeout_seconds=2.0,
                 combine_streaming=protocol)
    emap = workloads.round_robin_expert_map(experts, world)
    with EmulatedGroup(world, emap, cfg) as group:
        slot = group.create_slot()
        for seed in range(4):
            xs, ids, ws = [], [], []
            for rank in range(world):
                n = tokens if seed != 1 else max(tokens - 7 * rank, 0)          # uneven batches, one empty-ish
                i, w = (workloads.zipf_routing if seed == 3 else workloads.uniform_routing)(
                    n, experts, topk, seed=seed, rank=rank)
                xs.append(workloads.gaussian_payload(n, hidden, seed=seed, rank=rank))
                ids.append(i)
                ws.append(w)
            run_round(group, slot, xs, ids, ws, emap, direct_partial=(seed != 2), ctas=ctas,
                      rounding="two_step")


def test_a_short_partial_is_an_error_not_stale_data():
    """A rank whose partial tensor has fewer rows than it received cannot serve every owner: it
    reports a capacity error and the owners that wait for the missing rows stop with a status,
    instead of reducing whatever an earlier combine left in the staging rows."""
    world, hidden, topk, tokens = 2, 256, 2, 32
    cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=tokens, timeout_seconds=0.5)
    emap = workloads.round_robin_expert_map(4, world)
    with EmulatedGroup(world, emap, cfg) as group:
        slot = group.create_slot()
        dev = group.device
        routes = [workloads.uniform_routing(tokens, 4, topk, seed=1, rank=r) for r in range(world)]
        xs = [workloads.gaussian_payload(tokens, hidden, seed=1, rank=r).to(dev) for r in range(world)]
        batches = group.dispatch(slot, xs, [i.to(dev) for i, _ in routes], [w.to(dev) for _, w in routes])
        partials = [group.scale_rows(b) for b in batches]
        received = int(batches[0].valid_count.item())
        assert received > 8
        partials[0] = partials[0][:received - 5].clone()
        group.combine(slot, partials, [tokens] * world)
        statuses = [status[0] for status in group.status()]
        assert statuses[0] == 2 and statuses[1] in (3, 4)
        assert torch.ones(2, device=dev).sum().item() == 2   # the GPU is still usable


def test_mailbox_and_sequential_combine_agree_across_slots():
    """Two outstanding handles combined in reverse order, one mode per slot use."""
    world, hidden, topk, tokens = 4, 512, 4, 96
    experts = world * 2
    cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=tokens, timeout_seconds=2.0)
    emap = workloads.contiguous_expert_map(experts, world)
    with EmulatedGroup(world, emap, cfg) as group:
        dev = group.device
        slots = [group.create_slot(), group.create_slot()]
        outs = {}
        for mode in (1, 0):
            group.core.engine.set_combine_streaming(mode)
            batches = []
            for index, slot in enumerate(slots):
                xs = [workloads.gaussian_payload(tokens, hidden, seed=index, rank=r).to(dev) for r in range(world)]
                routes = [workloads.uniform_routing(tokens, experts, topk, seed=index, rank=r) for r in range(world)]
                batch = group.dispatch(slot, xs, [i.to(dev) for i, _ in routes], [w.to(dev) for _, w in routes])
                batches.append([group.scale_rows(b) for b in batch])
            for index in (1, 0):                                     # reverse order
                result = group.combine(slots[index], batches[index], [tokens] * world)
                outs[(mode, index)] = [o.clone() for o in result]
            assert all(status[0] == 0 for status in group.status())
        for index in (0, 1):
            for rank in range(world):
                assert torch.equal(bits(outs[(1, index)][rank]), bits(outs[(0, index)][rank]))


def test_random_delays_and_guard_bands_leave_results_exact():
    """Orderings shaken by per-CTA sleeps at every phase boundary; nothing lands outside a slot."""
    world, hidden, topk, tokens = 4, 512, 4, 150
    experts = world * 4
    cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=tokens, timeout_seconds=2.0,
                 diagnostics=True, debug_delay_ns=20000)
    emap = workloads.round_robin_expert_map(experts, world)
    with EmulatedGroup(world, emap, cfg) as group:
        slots = [group.create_slot(), group.create_slot()]
        assert all(slot.guards and len(slot.guards) == 2 * world for slot in slots)
        for seed in range(4):
            xs = [workloads.gaussian_payload(tokens, hidden, seed=seed, rank=r) for r in range(world)]
            routes = [workloads.uniform_routing(tokens, experts, topk, seed=seed, rank=r) for r in range(world)]
            run_round(group, slots[seed % 2], xs, [i for i, _ in routes], [w for _, w in routes], emap, ctas=6)
        group.check_guards()
        slots[1].guards[3][17] = 0                                 # what a stray store would do
        with pytest.raises(RuntimeError, match="guard band after the slot"):
            group.check_guards()
        slots[1].guards[3][17] = 0xA5
