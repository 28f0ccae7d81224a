"""One real rank against a peer that is played by the CPU, or that never shows up.

The group has two ranks but only rank 0 runs kernels; rank 1's heap exists so that rank 0's
stores have somewhere to land. The test writes (or withholds) rank 1's protocol words in rank
0's control region from the host - the reference's technique of forging words in a mapped
arena (tests/test_host_sm_native_cuda.py:109-125, :176-186). Every failure here is a wait that
runs out or a word the host forged; nothing faults or traps, and the GPU is used again after
each case.
"""

import pytest
import torch

from conftest import gpu_count

from ep_xpress_b200 import Config, native
from ep_xpress_b200.parallel.core import TransportCore

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(gpu_count() < 1, reason="needs a CUDA device")]

WORLD, HIDDEN, TOPK, TOKENS = 2, 128, 2, 12


class LoneRank:
    def __init__(self, timeout=0.05, diagnostics=False):
        self.m = native.load()
        self.cfg = Config(hidden_size=HIDDEN, topk=TOPK, max_tokens_per_rank=TOKENS, timeout_seconds=timeout,
                          diagnostics=diagnostics)
        self.bytes = self.cfg.heap_bytes(WORLD)
        self.heaps = [self.m.heap_allocate(self.bytes) for _ in range(WORLD)]
        # experts 0,1 live on rank 0, expert 2 on rank 1
        self.core = TransportCore(self.m, world=WORLD, local_ranks=[0], heaps=[self.heaps], heap_bytes=self.bytes,
                                  config=self.cfg, expert_to_rank=[0, 0, 1], device=torch.device("cuda", 0))
        self.slot = self.core.create_slot(WORLD * TOKENS, TOKENS)
        self.offsets = self.core.engine.ctrl_offsets()
        torch.cuda.synchronize()

    def forge_peer_dispatch_words(self, generation, *, count_for_me=0, identity=0):
        """What rank 1 would publish when it enters dispatch `generation` with nothing to send."""
        parity, tag = generation & 1, generation << 32
        poke = self.core.engine.poke_u64
        for dest, count in ((0, count_for_me), (1, 0)):
            poke(0, self.offsets["cnt"] + 8 * ((parity * WORLD + 1) * WORLD + dest), tag | count)
        peer_slot = self.slot.offsets[0]            # rank 1 "uses" the same layout in its own heap
        for k, value in enumerate((peer_slot >> 8, WORLD * TOKENS, WORLD * TOKENS, identity, 4)):   # 4 = its CTAs
            poke(0, self.offsets["addr"] + 8 * ((parity * WORLD + 1) * 8 + k), tag | value)

    def dispatch(self, ids, identity=0):
        x = torch.ones((TOKENS, HIDDEN), dtype=torch.bfloat16, device="cuda")
        w = torch.full((TOKENS, TOPK), 0.5, device="cuda")
        self.core.dispatch(self.slot, [x], [ids.cuda()], [w], [WORLD * TOKENS], identity=identity, ctas=4)
        torch.cuda.synchronize()
        return self.core.status(0)

    def close(self):
        torch.cuda.synchronize()
        self.core = None
        for heap in self.heaps:
            self.m.heap_release(heap)


LOCAL = torch.tensor([[0, 1]] * TOKENS)
MIXED = torch.tensor([[0, 2]] * TOKENS)


def usable():
    return torch.ones(2, device="cuda").sum().item() == 2


def test_absent_peer_runs_into_the_timeout_and_returns_control():
    rank = LoneRank(timeout=0.05)
    status, detail, dispatch_epoch, _ = rank.dispatch(LOCAL)
    assert status == 3 and dispatch_epoch == 0 and usable()       # timed out waiting, epoch not retired
    rank.close()


def test_cpu_played_peer_lets_a_local_dispatch_complete():
    rank = LoneRank(timeout=1.0)
    rank.forge_peer_dispatch_words(1)
    status, _, dispatch_epoch, _ = rank.dispatch(LOCAL)
    views = rank.slot.views[0]
    assert (status, dispatch_epoch) == (0, 1)
    assert int(views.count.item()) == TOKENS
    assert (views.local_ids[:TOKENS].cpu() == torch.tensor([0, 1])).all()
    assert (views.hidden[:TOKENS] == 1).all() and (views.hidden[TOKENS:] == 0).all()
    # rows for the peer really landed in ITS heap (rank 1's receive plane), none came back
    rank.forge_peer_dispatch_words(2)
    assert rank.dispatch(MIXED)[0] == 0
    peer_hidden = rank.m.Engine(WORLD, [1], HIDDEN, TOPK, [0, 0, 1], [rank.heaps], 1.0, False, 0).view(
        0, rank.slot.offsets[0] + rank.core.engine.layout(WORLD * TOKENS, TOKENS)["hidden"], [TOKENS, HIDDEN],
        torch.bfloat16)
    assert (peer_hidden == 1).all() and usable()
    rank.close()


def test_stale_generation_never_satisfies_a_wait():
    rank = LoneRank(timeout=0.05)
    for generation in (1, 2):
        rank.forge_peer_dispatch_words(generation)
        assert rank.dispatch(LOCAL)[0] == 0
    # Generation 3 shares its words with generation 1, whose values are still there.
    status, _, dispatch_epoch, _ = rank.dispatch(LOCAL)
    assert status == 3 and dispatch_epoch == 2 and usable()
    rank.close()


def test_a_peer_that_is_generations_ahead_is_reported_at_once():
    rank = LoneRank(timeout=5.0)
    rank.forge_peer_dispatch_words(3)                 # same parity as generation 1, but from the future
    begin = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    begin.record()
    status, detail, _, _ = rank.dispatch(LOCAL)
    end.record()
    torch.cuda.synchronize()
    assert status == 5 and (detail >> 32) & 0xff == 7 and detail & 0xffffffff == 1      # out of step with rank 1
    assert begin.elapsed_time(end) < 1000 and usable()
    rank.close()


def test_peer_error_word_aborts_the_wait_early():
    rank = LoneRank(timeout=5.0)
    rank.core.engine.poke_u64(0, rank.offsets["perr"], 3 << 32)   # u32 slot of rank 1 = code 3
    begin = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    begin.record()
    status = rank.dispatch(LOCAL)[0]
    end.record()
    torch.cuda.synchronize()
    assert status == 4 and begin.elapsed_time(end) < 1000 and usable()   # well before the 5 s timeout
    rank.close()


def test_identity_mismatch_is_detected_with_diagnostics():
    rank = LoneRank(timeout=1.0, diagnostics=True)
    rank.forge_peer_dispatch_words(1, identity=1234)
    assert rank.dispatch(LOCAL, identity=99)[0] == 5 and usable()
    rank.close()


def test_announced_rows_that_never_arrive_time_out_on_the_arrival_count():
    rank = LoneRank(timeout=0.05)
    rank.forge_peer_dispatch_words(1, count_for_me=3)  # the peer promises three rows; none of its CTAs ever counts in
    status, detail, _, _ = rank.dispatch(LOCAL)
    assert status == 3 and (detail >> 32) & 0xff == 6 and usable()
    rank.close()


def test_generations_never_wrap():
    """At the last usable generation the kernel refuses to run instead of reusing old tags."""
    rank = LoneRank(timeout=1.0)
    last = 0x7FFFFFFE
    rank.core.engine.poke_u64(0, 16, (last << 32) | last)        # disp_epoch and comb_epoch of the header
    status, detail, dispatch_epoch, combine_epoch = rank.dispatch(LOCAL)
    assert status == 6 and detail & 0xFFFFFFFF == last + 1
    assert (dispatch_epoch, combine_epoch) == (last, last) and usable()
    rank.close()


def test_cpu_played_peer_counts_its_ctas_in_and_the_counter_is_reset():
    """The peer announces rows and four CTAs; the wait ends when the arrival count reaches four
    (forged from the host before the launch), and the rank puts the counter back to zero."""
    rank = LoneRank(timeout=1.0)
    rank.forge_peer_dispatch_words(1, count_for_me=3)
    counter = rank.offsets["done"] + 8 * ((1 * WORLD) + 1)          # parity 1, source rank 1
    rank.core.engine.poke_u64(0, counter, 4)
    status, _, dispatch_epoch, _ = rank.dispatch(LOCAL)
    assert (status, dispatch_epoch) == (0, 1)
    assert rank.core.engine.peek_u64(0, counter) == 0 and usable()
    rank.close()
