"""CPU oracle self-tests, including the reference benchmark's first configuration:
2 simulated ranks, 8 experts round-robin, hidden 256, top-2, 64 tokens per rank, seed 0."""

import math

import pytest
import torch

from ep_xpress_b200.utils import routing, workloads


def roundtrip(world, experts, hidden, topk, tokens, seed, emap=None, rounding="two_step"):
    emap = workloads.round_robin_expert_map(experts, world) if emap is None else emap
    xs, ids, ws = [], [], []
    for rank in range(world):
        i, w = workloads.uniform_routing(tokens[rank], experts, topk, seed=seed, rank=rank)
        xs.append(workloads.gaussian_payload(tokens[rank], hidden, seed=seed, rank=rank))
        ids.append(i)
        ws.append(w)
    plan = routing.plan_routes(ids, ws, emap, world, topk)
    hidden_rows = routing.dispatch_oracle(xs, plan)
    partials = [routing.scale_expert_oracle(hidden_rows[r], plan.received[r].local_ids, plan.received[r].weights)
                for r in range(world)]
    out = routing.combine_oracle(partials, plan, hidden, rounding)
    direct = routing.direct_weighted_sum(xs, ids, ws)
    return plan, out, direct


def test_baseline_config_one():
    plan, out, direct = roundtrip(2, 8, 256, 2, [64, 64], seed=0)
    assert plan.token_counts == [64, 64]
    for rank in range(2):
        assert out[rank].shape == (64, 256)
        # weights sum to 1 and the expert is the identity: the output is x up to BF16 rounding steps
        assert torch.allclose(out[rank].to(torch.float64), direct[rank], rtol=2 ** -6, atol=2 ** -6)
        rows = plan.dest_rows[rank]
        assert ((rows >= 0).sum(dim=1) >= 1).all() and ((rows >= 0).sum(dim=1) <= 2).all()


@pytest.mark.parametrize("seed", range(12))
def test_randomised_round_trips(seed):
    g = torch.Generator().manual_seed(seed)
    world = int(torch.randint(1, 7, (1,), generator=g))
    topk = int(torch.randint(1, 5, (1,), generator=g))
    experts = world * int(torch.randint(1, 4, (1,), generator=g)) + topk
    emap = torch.randint(0, world, (experts,), generator=g).tolist()
    tokens = torch.randint(0, 20, (world,), generator=g).tolist()
    plan, out, direct = roundtrip(world, experts, 32, topk, tokens, seed, emap,
                                  rounding="single" if seed % 2 else "two_step")
    for rank in range(world):
        assert torch.allclose(out[rank].to(torch.float64), direct[rank], rtol=2 ** -5, atol=2 ** -5)


def test_dedup_and_order():
    emap = [0, 0, 1, 1]
    ids = [[[0, 1], [2, 0], [-1, -1]], [[3, 2]]]
    ws = [[[0.5, 0.5], [0.25, 0.75], [float("nan"), float("inf")]], [[0.5, 0.5]]]
    plan = routing.plan_routes(ids, ws, emap, 2, 2)
    assert plan.dest_masks[0].tolist() == [1, 3, 0]
    assert plan.dest_masks[1].tolist() == [2]
    assert plan.remote_masks()[0].tolist() == [0, 2, 0]
    r0, r1 = plan.received
    assert r0.inverse.tolist() == [[0, 0], [0, 1]]            # one row although both experts live on rank 0
    assert r0.local_ids.tolist() == [[0, 1], [-1, 0]]
    assert r1.inverse.tolist() == [[0, 1], [1, 0]]            # (source rank, token) order
    assert r1.local_ids.tolist() == [[0, -1], [1, 0]]
    assert r1.weights.tolist() == [[0.25, 0.75], [0.5, 0.5]]  # all active weights retained
    assert plan.dest_rows[0].tolist() == [[0, -1], [1, 0], [-1, -1]]


def test_dropped_slot_does_not_hide_an_active_slot_of_the_same_rank():
    plan = routing.plan_routes([[[0, 1, 2, -1]], []], [[[0.5, 0.25, 0.25, float("nan")]], []], [0, 0, 1, 1], 2, 4)
    assert plan.dest_masks[0].tolist() == [3]
    assert plan.received[1].local_ids.tolist() == [[-1, -1, 0, -1]]
    assert plan.received[1].weights.tolist() == [[0.5, 0.25, 0.25, 0.0]]


def test_local_ids_follow_order_of_appearance():
    assert routing.expert_local_ids([1, 0, 1, 1, 0], 2) == [0, 0, 1, 2, 1]


def test_wide_group_masks():
    world = 63
    emap = list(range(world))
    ids = [[[62, 0]]] + [[] for _ in range(world - 1)]
    ws = [[[0.5, 0.5]]] + [[] for _ in range(world - 1)]
    plan = routing.plan_routes(ids, ws, emap, world, 2)
    assert plan.dest_masks[0].tolist() == [(1 << 62) | 1]
    assert plan.received[62].rows == 1


@pytest.mark.parametrize("ids,ws,fragment", [
    ([[[0, 0]]], [[[0.5, 0.5]]], "same expert twice"),
    ([[[0, 4]]], [[[0.5, 0.5]]], "outside the supported range"),
    ([[[0, -2]]], [[[0.5, 0.5]]], "outside the supported range"),
    ([[[0, 1]]], [[[0.5, math.nan]]], "finite"),
    ([[[0, 1]]], [[[0.5, math.inf]]], "finite"),
])
def test_validation(ids, ws, fragment):
    with pytest.raises(ValueError, match=fragment):
        routing.plan_routes(ids + [[]], ws + [[]], [0, 1, 0, 1], 2, 2)


def test_rejects_malformed_groups():
    with pytest.raises(ValueError):
        routing.plan_routes([[]], [[]], [0], 64, 1)
    with pytest.raises(ValueError):
        routing.plan_routes([[]], [[]], [], 1, 1)
    with pytest.raises(ValueError):
        routing.plan_routes([[]], [[]], [1], 1, 1)
    with pytest.raises(ValueError):
        routing.plan_routes([[], []], [[]], [0], 1, 1)


def test_intermediate_rounding_is_observable():
    emap = [0, 1, 2]
    ids = [[[0, 1, 2]], [], []]
    ws = [[[1.0, 1.0, 1.0]], [], []]
    plan = routing.plan_routes(ids, ws, emap, 3, 3)
    parts = [torch.full((1, 4), v).to(torch.bfloat16) for v in (1.0, 2.0 ** -8, 2.0 ** -16)]
    two = routing.combine_oracle(parts, plan, 4, "two_step")[0]
    one = routing.combine_oracle(parts, plan, 4, "single")[0]
    assert not torch.equal(two, one)
