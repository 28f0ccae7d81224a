import dataclasses

import pytest

from ep_xpress_b200 import Config


def test_defaults_and_layout_helpers():
    cfg = Config(hidden_size=2048, topk=8, max_tokens_per_rank=4096)
    assert cfg.transport == "nvlink" and cfg.device_transport
    assert cfg.chunk_rows == (2 << 20) // 4096
    assert cfg.slot_bytes % 4096 == 0
    assert cfg.channel_chunk_rows(4) == 128
    assert cfg.combine_chunk_rows(4, 8) == 16
    assert cfg.heap_bytes(8) % (2 << 20) == 0
    assert cfg.heap_bytes(8) >= 2 * cfg.nvlink_slot_bytes(8)
    with pytest.raises(dataclasses.FrozenInstanceError):
        cfg.topk = 4


def test_slot_bytes_accounts_for_every_plane():
    cfg = Config(hidden_size=256, topk=2, max_tokens_per_rank=64)
    cap, tok = 128, 64
    minimum = cap * 256 * 2 * 2 + cap * 2 * 12 + cap * 16 + tok * 256 * 2
    assert cfg.nvlink_slot_bytes(2) >= minimum
    assert cfg.nvlink_slot_bytes(2, 10, 3) < cfg.nvlink_slot_bytes(2)


@pytest.mark.parametrize("kwargs,fragment", [
    (dict(diagnostics=1), "diagnostics must be a bool"),
    (dict(transport="host_ce", diagnostics=True), "only supported by host_sm"),
    (dict(transport="host_ce", decode_max_tokens=8), "only supported by host_sm"),
    (dict(decode_single_frame=True), "decode_single_frame"),
    (dict(channels=33), "channels must be at most 32"),
    (dict(hidden_size=0), "hidden_size must be a positive integer"),
    (dict(hidden_size=True), "hidden_size must be a positive integer"),
    (dict(hidden_size=7), "even hidden size"),
    (dict(topk=257), "topk <= 256"),
    (dict(timeout_seconds=float("inf")), "timeout_seconds"),
    (dict(timeout_seconds=4000.0), "3600"),
    (dict(workload="train"), "workload"),
    (dict(chunk_bytes=16), "chunk_bytes"),
    (dict(decode_max_tokens=257), "decode_max_tokens"),
    (dict(internode_transport="ib"), "internode_transport"),
    (dict(internode_transport="gin", transport="nvlink"), "GIN requires host_sm"),
    (dict(gin_contexts=0), "gin_contexts"),
    (dict(combine_rounding="banker"), "combine_rounding"),
])
def test_validation(kwargs, fragment):
    base = dict(hidden_size=64, topk=2, max_tokens_per_rank=8)
    base.update(kwargs)
    with pytest.raises(ValueError, match=fragment):
        Config(**base)


@pytest.mark.parametrize("kwargs", [dict(transport="rdma"), dict(combine_backend="cpu"), dict(graph_mode="capture")])
def test_not_implemented(kwargs):
    with pytest.raises(NotImplementedError):
        Config(hidden_size=64, topk=2, max_tokens_per_rank=8, **kwargs)


def test_host_ce_allows_odd_hidden_and_reports_host_pool():
    cfg = Config(hidden_size=7, topk=2, max_tokens_per_rank=8, transport="host_ce")
    assert cfg.pool_bytes(4) > 0
    assert cfg.pinned_working_set_bytes(4) > cfg.pool_bytes(4)
    assert Config(hidden_size=64, topk=2, max_tokens_per_rank=8).pool_bytes(4) == 0


def test_gin_selects_the_multinode_context_and_single_rounding():
    from ep_xpress_b200 import Context
    cfg = Config(hidden_size=64, topk=2, max_tokens_per_rank=8, transport="host_sm", internode_transport="gin")
    assert cfg.single_rounding and not Config(hidden_size=64, topk=2, max_tokens_per_rank=8).single_rounding
    assert not Config(hidden_size=64, topk=2, max_tokens_per_rank=8, transport="host_sm", internode_transport="gin",
                      combine_rounding="two_step").single_rounding
    with pytest.raises(TypeError, match="NCCLCommHandle"):
        Context(None, [0], cfg)                                     # the multi-node context checks its communicator


def test_multinode_sizing_helpers_follow_the_record_layout():
    cfg = Config(hidden_size=256, topk=2, max_tokens_per_rank=64, transport="host_sm", internode_transport="gin")
    record = 640                                   # 512 B row + 16 B ids/weights + 4 B token -> 128-byte units
    records = (128 + 64 * record + 4095) // 4096 * 4096
    assert cfg.gin_producer_bytes(4) == (records + 4 * 64 * 512 + 4095) // 4096 * 4096
    granule = 2 << 20
    raw = 128 + (16 + 1) * 64 * record + 16 * 64 * 256 * 4
    assert cfg.gin_registered_bytes(16) == (raw + granule - 1) // granule * granule
    assert cfg.pool_bytes(16, local_world_size=4) == 4 * cfg.gin_producer_bytes(4)
    with pytest.raises(ValueError, match="local_world_size < world_size"):
        cfg.pool_bytes(16, local_world_size=16)
    with pytest.raises(ValueError, match=r"\[2, 256\]"):
        cfg.gin_registered_bytes(1)
    with pytest.raises(ValueError, match=r"\[1, 256\]"):
        cfg.gin_producer_bytes(True)


def test_mapped_arena_is_empty_but_validated():
    cfg = Config(hidden_size=256, topk=2, max_tokens_per_rank=64)
    assert cfg.mapped_arena_bytes(2) == 0 and cfg.mapped_arena_bytes(0, queue_peers=8) == 0
    with pytest.raises(ValueError, match="dispatch_banks"):
        cfg.mapped_arena_bytes(2, dispatch_banks=1)
    with pytest.raises(ValueError, match="only valid for dispatch"):
        cfg.mapped_arena_bytes(0, dispatch_banks=2)
    with pytest.raises(ValueError, match="queue_peers"):
        cfg.mapped_arena_bytes(2, queue_peers=2)


def test_inert_fields_are_named_and_slot_breakdown_adds_up():
    cfg = Config(hidden_size=512, topk=4, max_tokens_per_rank=64)
    assert cfg.inert_fields() == ()
    noisy = Config(hidden_size=512, topk=4, max_tokens_per_rank=64, chunk_bytes=1 << 20, decode_max_tokens=32,
                   decode_single_frame=True, combine_warp_specialization=True, workload="decode")
    assert set(noisy.inert_fields()) == {"chunk_bytes", "decode_single_frame", "combine_warp_specialization", "workload"}
    assert Config(hidden_size=512, topk=4, max_tokens_per_rank=64, transport="host_ce", chunk_bytes=1 << 20).inert_fields() == ()
    for world in (1, 3, 8):
        parts = cfg.nvlink_slot_breakdown(world)
        assert parts["total"] == cfg.nvlink_slot_bytes(world)
        assert parts["staging"] >= 64 * min(4, world) * (512 * 2 + 128)
