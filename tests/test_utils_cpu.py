"""Harness utilities on CPU: clock sampler against a fake NVML, profile decoding, workloads."""

import sys
import time
import types
from types import SimpleNamespace
from unittest import mock

import pytest
import torch

from ep_xpress_b200.utils import clocks, profile, routing, workloads


def fake_nvml(clock_values, reason_bits):
    module = types.ModuleType("pynvml")
    state = {"reads": 0}
    module.NVML_CLOCK_SM = 1
    module.nvmlInit = lambda: None
    module.nvmlDeviceGetHandleByIndex = lambda index: ("gpu", index)
    module.nvmlDeviceGetMaxClockInfo = lambda handle, kind: 1965

    def clock(handle, kind):
        state["reads"] += 1
        return clock_values[min(state["reads"] - 1, len(clock_values) - 1)]
    module.nvmlDeviceGetClockInfo = clock
    module.nvmlDeviceGetCurrentClocksEventReasons = lambda handle: reason_bits

    def refuse(name):
        raise AssertionError(f"the sampler must never call {name}")
    for setter in ("nvmlDeviceSetGpuLockedClocks", "nvmlDeviceResetGpuLockedClocks", "nvmlDeviceSetPowerManagementLimit",
                   "nvmlDeviceSetPersistenceMode", "nvmlDeviceSetApplicationsClocks"):
        setattr(module, setter, lambda *a, name=setter: refuse(name))
    module.state = state
    return module


def test_clock_sampler_reads_and_never_writes():
    nvml = fake_nvml([1965, 1965, 1800], 0x4 | 0x20)
    with mock.patch.dict(sys.modules, {"pynvml": nvml}):
        sampler = clocks.ClockSampler(0, interval_s=0.001)
        with sampler:
            deadline = time.time() + 2.0
            while len(sampler.samples) < 5 and time.time() < deadline:
                time.sleep(0.002)
            sampler.pause()
            time.sleep(0.01)
            frozen = len(sampler.samples)
            time.sleep(0.02)
            assert len(sampler.samples) <= frozen + 1              # paused: at most the sample in flight
        summary = sampler.summary()
    assert summary["sm_max_mhz"] == 1965 and summary["samples"] >= 5
    assert summary["sm_mhz"] in (1800, 1965)
    assert summary["reasons"] == ["sw_power_cap", "sw_thermal_slowdown"]


def test_clock_sampler_without_nvml_reports_instead_of_failing():
    broken = types.ModuleType("pynvml")

    def init():
        raise RuntimeError("no driver")
    broken.nvmlInit = init
    with mock.patch.dict(sys.modules, {"pynvml": broken}):
        with clocks.ClockSampler(0) as sampler:
            pass
    summary = sampler.summary()
    assert summary["sm_mhz"] is None and "no driver" in summary["error"]


@pytest.fixture()
def profiled_context():
    context = SimpleNamespace(device=torch.device("cpu"), rank=3,
                              _core=SimpleNamespace(native=SimpleNamespace(PROFILE_STAMPS=8), max_ctas=4))
    stream = SimpleNamespace(synchronize=lambda: None)
    with mock.patch.object(torch.cuda, "is_current_stream_capturing", lambda: False), \
            mock.patch.object(torch.cuda, "current_stream", lambda device=None: stream), \
            mock.patch.object(torch.Tensor, "pin_memory", lambda self: self):
        yield context


def test_operation_profile_decodes_stamps_and_counts_drops(profiled_context):
    session = profile.OperationProfile(profiled_context, max_operations=2)
    session.label = "warm"
    first = session.slice_for("dispatch", 7, "tag", 12, 24, 2)
    first[0, :8] = torch.tensor([1000, 1100, 1200, 1300, 1400, 1500, 1600, 1700])
    first[1, :8] = torch.tensor([1010, 1150, 1250, 1350, 1450, 1550, 0, 0])         # this CTA stopped early
    second = session.slice_for("combine", 7, None, 12, 24, 1)
    second[0, :8] = torch.tensor([5000, 5400, 5500, 5900, 11, 22, 33, 44])
    assert session.slice_for("dispatch", 8, None, 1, 1, 1) is None                    # full: dropped
    report = session.finish()
    assert report["rank"] == 3 and report["dropped_operations"] == 1 and len(report["operations"]) == 2
    dispatch, combine = report["operations"]
    assert dispatch["label"] == "warm" and dispatch["phases"]["start"] == {"first_ns": 0, "last_ns": 10}
    assert dispatch["phases"]["routed"] == {"first_ns": 100, "last_ns": 150}
    assert dispatch["phases"]["done"] == {"first_ns": 700, "last_ns": 700} and dispatch["elapsed_ns"] == 700
    assert combine["phases"]["reduced"] == {"first_ns": 900, "last_ns": 900}
    assert combine["cycles"]["consumer_wait_cycles"] == 11 and combine["cycles"]["producer_other_cycles"] == 44


def test_wide_profile_records_give_disjoint_phases_that_sum_to_elapsed():
    """24-word records: per-CTA phases between consecutive stamps, counters, milestones, invariants."""
    record = {"kind": "dispatch", "operation": 3, "tag": None, "label": None, "tokens": 8, "capacity": 16, "ctas": 2}
    stamps = torch.zeros((2, 24), dtype=torch.int64)
    stamps[0, :8] = torch.tensor([1000, 1100, 1200, 1300, 1900, 1950, 1960, 2000])
    stamps[1, :8] = torch.tensor([1010, 1020, 1210, 1310, 1800, 1900, 1900, 2040])
    stamps[:, profile.WORDS["rows"]] = torch.tensor([5, 7])
    stamps[:, profile.WORDS["bytes"]] = torch.tensor([5 * 512, 7 * 512])
    stamps[:, profile.WORDS["polls"]] = torch.tensor([40, 2])
    stamps[0, profile.WORDS["first_publish"]] = 1005
    stamps[:, profile.WORDS["first_receive"]] = torch.tensor([1290, 1305])
    stamps[:, profile.WORDS["completion"]] = 7
    stamps[:, profile.WORDS["mode"]] = 2
    entry = profile.summarize(record, stamps)
    assert entry["protocol"] == "bulk" and entry["rows"] == 12 and entry["bytes"] == 12 * 512 and entry["polls"] == 42
    assert entry["first_publish_ns"] == 5 and entry["first_receive_ns"] == 290
    assert entry["cta_phase_ns"]["payload"] == [600, 490] and entry["cta_elapsed_ns"] == [1000, 1030]
    assert list(entry["cta_phase_ns"]) == list(profile.DISPATCH_INTERVALS)
    profile.check_invariants(entry, row_bytes=512)
    stamps[1, profile.WORDS["completion"]] = 4                       # a CTA that never finished
    with pytest.raises(AssertionError):
        profile.check_invariants(profile.summarize(record, stamps))
    mailbox = {"kind": "combine", "operation": 3, "tag": None, "label": None, "tokens": 8, "capacity": 16, "ctas": 1}
    stamps = torch.zeros((1, 24), dtype=torch.int64)
    stamps[0, :4] = torch.tensor([500, 0, 900, 950])                 # this CTA's pusher found no row
    stamps[0, profile.WORDS["completion"]] = 3
    stamps[0, profile.WORDS["mode"]] = 3
    entry = profile.summarize(mailbox, stamps)
    assert entry["protocol"] == "mailbox" and entry["cta_phase_ns"]["retire"] == [50]
    assert sum(v[0] for v in entry["cta_phase_ns"].values()) == entry["cta_elapsed_ns"][0] == 450
    profile.check_invariants(entry)


def test_operation_profile_budget_and_arguments(profiled_context):
    with pytest.raises(ValueError, match="64 MiB budget"):
        profile.OperationProfile(profiled_context, max_operations=(64 << 20) // (4 * 8 * 8) + 1)
    with pytest.raises(ValueError, match="max_operations"):
        profile.OperationProfile(profiled_context, max_operations=0)
    with mock.patch.object(torch.cuda, "is_current_stream_capturing", lambda: True):
        assert profile.OperationProfile(profiled_context, 4).slice_for("dispatch", 1, None, 1, 1, 1) is None


def test_replay_cases_have_their_defining_properties():
    world, tokens, topk = 4, 12, 4
    ids, weights, experts = workloads.replay_case("mixed", rank=1, world_size=world, tokens=tokens, topk=topk)
    assert experts == 16 and ids.shape == (tokens, topk)
    owners = ids // 4
    assert (owners[:, 0] == owners[:, 1]).all() and (owners[:, 2] == owners[:, 3]).all()   # pairs share a rank
    assert workloads.replay_case("empty", rank=world - 1, world_size=world, tokens=tokens)[0].shape[0] == 0
    assert workloads.replay_case("empty", rank=2, world_size=world, tokens=tokens)[0].shape[0] == tokens - 2
    assert (workloads.replay_case("hotspot", rank=3, world_size=world, tokens=tokens)[0] // 4 == 0).all()
    assert (workloads.replay_case("local", rank=3, world_size=world, tokens=tokens)[0] // 4 == 3).all()
    ids, weights, _ = workloads.replay_case("padding", rank=0, world_size=world, tokens=tokens)
    assert (ids[0] == -1).all() and torch.isnan(weights[0]).all()
    assert ids[1, -1] == -1 and torch.isinf(weights[1, -1]) and (ids[2] >= 0).all()
    assert (workloads.replay_case("all_padding", rank=0, world_size=world, tokens=tokens)[0] == -1).all()
    with pytest.raises(ValueError, match="unknown case"):
        workloads.replay_case("nope", rank=0, world_size=world, tokens=1)


def test_marker_payload_is_exact_in_bf16():
    x = workloads.marker_payload(300, 16, rank=5, iteration=9).float()
    assert (x[:, 0] == 5).all() and (x[:, 4] == 9).all()
    assert x[129, 1] == 1 and x[129, 2] == 1 and x[299, 1] == 299 % 128 and x[299, 2] == 2


def test_zipf_routing_is_skewed_and_without_replacement():
    ids, weights = workloads.zipf_routing(4096, 128, 8, seed=0, rank=0)
    assert ids.shape == (4096, 8) and weights.shape == (4096, 8)
    assert all(len(set(row.tolist())) == 8 for row in ids[:64])
    counts = torch.bincount(ids.flatten(), minlength=128).float()
    assert counts.max() > 6 * counts.mean()                       # a hot expert far above the uniform share
    assert torch.allclose(weights.sum(dim=1), torch.ones(4096), atol=1e-5)
    again, _ = workloads.zipf_routing(4096, 128, 8, seed=0, rank=1)
    assert counts.argmax() == torch.bincount(again.flatten(), minlength=128).argmax()   # same popularity on every rank


def test_communication_patterns_rotate():
    kwargs = dict(rank=2, world_size=4, tokens=30, num_experts=16, topk=4)
    random_ids, w = workloads.communication_pattern(0, **kwargs)
    assert (w == 0.25).all() and all(len(set(row.tolist())) == 4 for row in random_ids)
    hot, _ = workloads.communication_pattern(5, **kwargs)                # 5 % 4 == 1: everything to rank 5 % 4
    assert (hot * 4 // 16 == 1).all() and (hot == hot[0]).all()
    dropped, _ = workloads.communication_pattern(2, **kwargs)
    assert (dropped[::3] == -1).all() and (dropped[1::3] >= 0).all()
    empty, _ = workloads.communication_pattern(0, rank=0, world_size=4, tokens=0, num_experts=16, topk=4)
    assert empty.shape == (0, 4)


@pytest.mark.parametrize("rounding", ["two_step", "single"])
@pytest.mark.parametrize("world", [1, 2, 4])
def test_identity_layer_oracle_matches_the_group_wide_oracles(world, rounding):
    """The per-rank shortcut the benchmarks verify against equals dispatch -> weighted identity
    expert -> combine computed over the whole group's route plan, bit for bit."""
    torch.manual_seed(3)
    experts, topk, hidden, tokens = 12, 4, 64, 23
    owners = workloads.round_robin_expert_map(experts, world)
    routes = [workloads.uniform_routing(tokens - r, experts, topk, seed=5, rank=r, weights="sigmoid") for r in range(world)]
    ids, ws = [i.clone() for i, _ in routes], [w for _, w in routes]
    ids[0][3, 1] = -1                                   # an inactive slot
    xs = [workloads.gaussian_payload(tokens - r, hidden, seed=7, rank=r) for r in range(world)]
    plan = routing.plan_routes(ids, ws, owners, world, topk)
    rows = routing.dispatch_oracle(xs, plan)
    partials = [routing.scale_expert_oracle(rows[r], plan.received[r].local_ids, plan.received[r].weights)
                for r in range(world)]
    want = routing.combine_oracle(partials, plan, hidden, rounding)
    for rank in range(world):
        got = routing.identity_layer_oracle(xs[rank], ids[rank], ws[rank], owners, rank, world, rounding)
        assert torch.equal(got.view(torch.int16), want[rank].view(torch.int16))


def test_identity_layer_oracle_property():
    """Random shapes, placements, inactive slots and zero weights: the per-rank shortcut and the
    group-wide oracles agree bit for bit (hypothesis drives the cases)."""
    hypothesis = pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=40, deadline=None)
    @given(world=st.integers(1, 5), experts_per_rank=st.integers(1, 3), topk=st.integers(1, 4),
           tokens=st.integers(0, 9), seed=st.integers(0, 10_000), rounding=st.sampled_from(["two_step", "single"]))
    def check(world, experts_per_rank, topk, tokens, seed, rounding):
        experts = world * experts_per_rank
        topk = min(topk, experts)
        generator = torch.Generator().manual_seed(seed)
        owners = torch.randint(0, world, (experts,), generator=generator).tolist()
        xs, ids, ws = [], [], []
        for rank in range(world):
            n = max(tokens - rank, 0)
            scores = torch.rand((n, experts), generator=generator)
            chosen = scores.topk(topk, dim=1).indices.to(torch.int64)
            chosen[torch.rand((n, topk), generator=generator) < 0.15] = -1
            weights = torch.rand((n, topk), generator=generator)
            weights[torch.rand((n, topk), generator=generator) < 0.1] = 0.0
            xs.append(torch.randn((n, 16), generator=generator).to(torch.bfloat16))
            ids.append(chosen)
            ws.append(weights)
        plan = routing.plan_routes(ids, ws, owners, world, topk)
        rows = routing.dispatch_oracle(xs, plan)
        partials = [routing.scale_expert_oracle(rows[r], plan.received[r].local_ids, plan.received[r].weights)
                    for r in range(world)]
        want = routing.combine_oracle(partials, plan, 16, rounding)
        for rank in range(world):
            got = routing.identity_layer_oracle(xs[rank], ids[rank], ws[rank], owners, rank, world, rounding)
            assert torch.equal(got.view(torch.int16), want[rank].view(torch.int16))

    check()
