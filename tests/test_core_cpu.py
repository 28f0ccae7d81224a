"""Heap carving and Python/native layout agreement (no GPU: only host functions of the runtime)."""

import pytest

from ep_xpress_b200 import Config, native
from ep_xpress_b200.parallel.core import HeapAllocator, TransportCore


def test_allocator_first_fit_coalescing_and_exhaustion():
    heap = HeapAllocator(4096, 4096 + 10 * 4096)
    a = heap.allocate(4096)
    b = heap.allocate(2 * 4096 - 1)          # rounded up to whole pages
    c = heap.allocate(4096)
    assert (a, b, c) == (4096, 8192, 16384)
    heap.release(b)
    assert heap.allocate(4096) == 8192      # first fit reuses the hole
    heap.release(a)
    heap.release(8192)
    assert heap.allocate(3 * 4096) == 4096  # neighbouring holes were merged
    assert heap.free_bytes == 6 * 4096
    with pytest.raises(MemoryError, match="workspace_pool_bytes"):
        heap.allocate(7 * 4096)
    with pytest.raises(KeyError):
        heap.release(12345)
    with pytest.raises(ValueError):
        HeapAllocator(100, 4096)


@pytest.mark.parametrize("hidden,topk,tokens,world", [(256, 2, 64, 2), (7168, 8, 4096, 8), (258, 3, 17, 5),
                                                      (2048, 33, 100, 63), (64, 1, 1, 1)])
def test_python_layout_mirrors_the_native_layout(hidden, topk, tokens, world):
    m = native.load()
    cfg = Config(hidden_size=hidden, topk=topk, max_tokens_per_rank=tokens)
    assert m.ctrl_bytes(world) == cfg.ctrl_bytes(world)
    assert m.slot_bytes(world * tokens, tokens, hidden, topk, world) == cfg.nvlink_slot_bytes(world)
    assert m.slot_bytes(10, 3, hidden, topk, world) == cfg.nvlink_slot_bytes(world, 10, 3)
    assert cfg.heap_bytes(world) >= cfg.ctrl_bytes(world) + cfg.slots * cfg.nvlink_slot_bytes(world)


def test_expert_runner_bounds():
    m = native.load()
    assert m.moe_sizes(1024, 8, 32) == (12288, 96)
    assert m.moe_sizes(1024, 8, 32, 256) == ((8192 // 256 + 32) * 256, 64)
    assert m.moe_sizes(10, 8, 2)[1] == 1 + 2            # at most min(topk, experts) local slots per row


def test_build_identity_is_stable_and_lazy_import_does_not_touch_cuda():
    import subprocess
    import sys
    assert native.build_identity() == native.build_identity()
    code = ("import sys, ep_xpress_b200; assert 'torch' not in sys.modules; "
            "assert 'ep_xpress_b200.native' not in sys.modules; print(ep_xpress_b200.__all__)")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr


def test_launch_width_follows_items_per_cta():
    core = object.__new__(TransportCore)
    core.hidden, core.max_ctas, core.items_per_cta = 7168, 148, 4
    # dispatch: one mover warp per row (four per CTA) until the budget is reached
    assert core.pick_ctas(128) == 32 and core.pick_ctas(4096) == 148 and core.pick_ctas(1) == 1
    assert core.pick_ctas(128, budget=30) == 30 and core.pick_ctas(0) == 1
    core.items_per_cta = 1
    assert core.pick_ctas(8) == 8 and core.pick_ctas(128) == 128
    core.hidden = 16384                       # rows of 32 KiB move as three pieces
    assert core.pick_ctas(8) == 24
    # combine: six received rows per CTA, at least one CTA per token and two CTAs in all
    assert core.pick_combine_ctas(128, 1024) == 148 and core.pick_combine_ctas(1, 8) == 2
    assert core.pick_combine_ctas(16, 16) == 16 and core.pick_combine_ctas(4096, 32768, budget=100) == 100
    assert core.pick_combine_ctas(1, 1) == 2 and core.pick_combine_ctas(8, 64) == 11
    # with peers, the tiniest batch still gets one pusher per fifteen interleaved work items
    core.world = 8
    assert core.pick_combine_ctas(1, 8) == 10 and core.pick_combine_ctas(8, 64) == 11
    core.world = 4
    assert core.pick_combine_ctas(1, 4) == 5
    core.world = 2
    assert core.pick_combine_ctas(1, 2) == 3


def test_load_refuses_a_binary_built_from_other_sources(monkeypatch):
    """The stamp names the sources a library was built from: a mismatch is never imported."""
    from ep_xpress_b200 import native
    monkeypatch.setattr(native, "_module", None)
    monkeypatch.setattr(native, "source_identity", lambda: "0123456789abcdef")
    monkeypatch.setattr(native.shutil, "which", lambda name: None)
    assert not native.is_built()
    with pytest.raises(RuntimeError, match="built from other sources"):
        native.load()
    rebuilt = []
    monkeypatch.setattr(native.shutil, "which", lambda name: "/usr/local/cuda/bin/nvcc")
    monkeypatch.setattr(native, "build", lambda **kwargs: rebuilt.append(True) or (_ for _ in ()).throw(RuntimeError("stop")))
    with pytest.raises(RuntimeError, match="stop"):
        native.load()                                # with a compiler present it rebuilds instead
    assert rebuilt == [True]
