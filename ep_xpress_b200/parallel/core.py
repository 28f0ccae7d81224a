"""Rank-local runtime of the NVLink transport: heap carving, slots, launches.

``TransportCore`` owns the native prepared operator and the slots carved out
of this process's peer-mapped heap(s). It drives ONE rank in production
(:class:`~ep_xpress_b200.parallel.nvlink.NVLinkContext`) or all ranks of a group
that share one GPU inside single cooperative launches
(:class:`~ep_xpress_b200.parallel.emulated.EmulatedGroup`).

A *slot* is the unit of storage of one dispatch/combine pair: the receive
planes peers store into, the partial plane peers load from, and local route
state. The reference allocates the equivalent tensors per operation or in a
``HostSMWorkspace`` (ep_xpress/host_sm.py:128-169, :1033-1053); here they are
fixed regions of the heap, so every address is stable across CUDA graph
replays and nothing is allocated on the hot path.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch

_ALIGN = 4096
_GUARD_BYTES = 4096        # keeps the slot itself page-aligned
_GUARD_PATTERN = 0xA5


class HeapAllocator:
    """First-fit allocator with coalescing over ``[start, end)`` of a heap."""

    def __init__(self, start: int, end: int):
        if start % _ALIGN or end <= start:
            raise ValueError("heap range must be aligned and non-empty")
        self._free = [(start, end)]
        self._live = {}

    def allocate(self, size: int) -> int:
        size = (size + _ALIGN - 1) // _ALIGN * _ALIGN
        for index, (begin, end) in enumerate(self._free):
            if end - begin >= size:
                if end - begin == size:
                    del self._free[index]
                else:
                    self._free[index] = (begin + size, end)
                self._live[begin] = size
                return begin
        raise MemoryError(
            f"the peer-mapped heap has no free range of {size} bytes; raise Config.workspace_pool_bytes "
            "or release workspaces")

    def release(self, offset: int) -> None:
        size = self._live.pop(offset)
        self._free.append((offset, offset + size))
        self._free.sort()
        merged = []
        for begin, end in self._free:
            if merged and merged[-1][1] == begin:
                merged[-1] = (merged[-1][0], end)
            else:
                merged.append((begin, end))
        self._free = merged

    @property
    def free_bytes(self) -> int:
        return sum(end - begin for begin, end in self._free)


@dataclass(repr=False)
class SlotViews:
    """Tensor views of one rank's slot (no copies; storage is the heap)."""
    hidden: torch.Tensor       # bf16  [capacity, hidden]
    local_ids: torch.Tensor    # int64 [capacity, topk]
    weights: torch.Tensor      # f32   [capacity, topk]
    inverse: torch.Tensor      # int64 [capacity, 2]
    partial: torch.Tensor      # bf16  [capacity, hidden]
    count: torch.Tensor        # int32 [1]  valid_count
    mask: torch.Tensor         # int64 [tokens]  destination-rank set per local token
    dest_rows: torch.Tensor    # int32 [tokens, fanout]  row index at the j-th destination rank
    send_counts: torch.Tensor  # int32 [world]
    recv_counts: torch.Tensor  # int32 [world]
    output: torch.Tensor       # bf16  [tokens, hidden]


@dataclass(repr=False, eq=False)      # identity semantics: slots are looked up in lists
class Slot:
    capacity: int
    tokens: int
    offsets: List[int]                 # heap offset per local rank
    views: List[SlotViews]
    generation: int = 0                # dispatches that used this slot
    busy: bool = False                 # dispatched, combine not yet enqueued
    released: bool = False
    tag: object = field(default=None, repr=False)
    bases: Optional[List[int]] = None  # allocation start per local rank when guard bands surround the slot
    guards: Optional[List[torch.Tensor]] = None   # uint8 views of the guard bands (diagnostics)


class TransportCore:
    def __init__(self, native, *, world, local_ranks, heaps, heap_bytes, config, expert_to_rank, device):
        self.native = native
        self.world = world
        self.local_ranks = list(local_ranks)
        self.config = config
        self.device = torch.device(device)
        self.hidden, self.topk = config.hidden_size, config.topk
        self.engine = native.Engine(world, self.local_ranks, self.hidden, self.topk, list(expert_to_rank),
                                    [list(map(int, row)) for row in heaps], float(config.timeout_seconds),
                                    config.single_rounding, self.device.index,
                                    bool(config.cooperative_launch))
        self.engine.set_combine_streaming({"auto": -1, "off": 0, "on": 1}[config.combine_streaming])
        if config.debug_delay_ns:
            self.engine.set_debug_delay(int(config.debug_delay_ns))
        ctrl = self.engine.ctrl_bytes()
        self._allocators = [HeapAllocator(ctrl, heap_bytes) for _ in self.local_ranks]
        self.max_ctas = max(1, min(self.engine.max_ctas(config.max_tokens_per_rank), self.engine.sm_count()))
        self.items_per_cta = 4            # rows a CTA of the dispatch kernel should find (one per mover warp)
        self.launches = 0
        self._slots: List[Slot] = []

    # ---- slots ---------------------------------------------------------------
    def create_slot(self, capacity: int, tokens: int, stream=None) -> Slot:
        layout = self.engine.layout(capacity, tokens)
        stream = stream or torch.cuda.current_stream(self.device)
        fanout = min(self.topk, self.world)
        offsets, views = [], []
        # Diagnostics: a band of a known byte pattern before and after every slot. Nothing may
        # ever write there, so `check_guards` turns a stray peer store (a wrong row index, a
        # stale slot address) into a reported error instead of silent corruption next door.
        guarded = bool(self.config.diagnostics)
        bases, guards = [], []
        for local, allocator in enumerate(self._allocators):
            if guarded:
                base = allocator.allocate(layout["bytes"] + 2 * _GUARD_BYTES)
                offset = base + _GUARD_BYTES
                for at in (base, offset + layout["bytes"]):
                    band = self.engine.view(local, at, [_GUARD_BYTES], torch.uint8)
                    with torch.cuda.stream(stream):
                        band.fill_(_GUARD_PATTERN)
                    guards.append(band)
            else:
                base = offset = allocator.allocate(layout["bytes"])
            bases.append(base)
            offsets.append(offset)
            self.engine.slot_reset(local, offset, capacity, tokens, stream.cuda_stream)

            def view(name, shape, dtype, local=local, offset=offset):
                return self.engine.view(local, offset + layout[name], list(shape), dtype)

            views.append(SlotViews(
                hidden=view("hidden", (capacity, self.hidden), torch.bfloat16),
                local_ids=view("ids", (capacity, self.topk), torch.int64),
                weights=view("weights", (capacity, self.topk), torch.float32),
                inverse=view("inverse", (capacity, 2), torch.int64),
                partial=view("partial", (capacity, self.hidden), torch.bfloat16),
                count=view("misc", (1,), torch.int32),
                mask=view("mask", (tokens,), torch.int64),
                dest_rows=view("send_rows", (tokens, fanout), torch.int32),
                send_counts=view("send_cnt", (self.world,), torch.int32),
                recv_counts=view("recv_cnt", (self.world,), torch.int32),
                output=view("output", (tokens, self.hidden), torch.bfloat16),
            ))
        slot = Slot(capacity, tokens, offsets, views, bases=bases, guards=guards if guarded else None)
        self._slots.append(slot)
        return slot

    def release_slot(self, slot: Slot) -> None:
        if slot.released:
            return
        slot.released = True
        if slot in self._slots:
            self._slots.remove(slot)
        for allocator, offset in zip(self._allocators, slot.bases or slot.offsets):
            allocator.release(offset)

    def check_guards(self) -> None:
        """Raise if any guard band around a live slot was written to (diagnostics only)."""
        for slot in self._slots:
            for index, band in enumerate(slot.guards or ()):
                if not bool((band == _GUARD_PATTERN).all()):
                    where = "before" if index % 2 == 0 else "after"
                    raise RuntimeError(f"guard band {where} the slot at heap offset {slot.offsets[index // 2]} of local "
                                       f"rank {index // 2} was overwritten: a store landed outside its slot")

    # ---- launches --------------------------------------------------------------
    def pick_ctas(self, tokens: int, budget: Optional[int] = None) -> int:
        """CTAs per rank of a dispatch: one mover warp per row piece until the budget is reached."""
        budget = self.max_ctas if budget is None else max(1, min(budget, self.max_ctas))
        pieces = -(-self.hidden * 2 // 14336)
        wanted = -(-max(tokens, 1) * pieces // max(1, self.items_per_cta))
        return max(1, min(budget, wanted))

    def pick_combine_ctas(self, tokens: int, capacity: int, budget: Optional[int] = None) -> int:
        """CTAs per rank of a combine. Under the mailbox protocol 7/16 of them (at most 64) only
        push - fifteen received rows per round trip each - and the others reduce four (token, row
        segment) items at a time; small batches get enough CTAs for one round trip to move
        everything (one round per pusher also for the tiniest batch), and never fewer than two (one
        pushes, one reduces)."""
        budget = self.max_ctas if budget is None else max(1, min(budget, self.max_ctas))
        # The pushers walk the received rows interleaved over the peers in blocks of eight, holes
        # included: even one row per peer is (world - 1) * 8 work items, fifteen per pusher round.
        peers = max(getattr(self, "world", 1) - 1, 0)
        pushers = -(-peers * 8 // 15)
        floor = max(2, -(-pushers * 16 // 7))
        wanted = max(floor, -(-max(capacity, 1) // 6), max(tokens, 1))
        return max(1, min(budget, wanted))

    def dispatch(self, slot: Slot, xs, ids, weights, capacities, *, identity=0, ctas=None, stream=None,
                 profile=None, samples=None):
        stream = stream or torch.cuda.current_stream(self.device)
        tokens = max(x.shape[0] for x in xs)
        ctas = self.pick_ctas(tokens) if ctas is None else ctas
        n = len(self.local_ranks)
        self.engine.dispatch(list(xs), list(ids), list(weights), slot.offsets, list(capacities),
                             [slot.capacity] * n, [slot.tokens] * n, identity, ctas,
                             bool(self.config.zero_padding), stream.cuda_stream, profile, samples)
        self.launches += 1

    def combine(self, slot: Slot, partials, outs, *, identity=0, ctas=None, stream=None, profile=None,
                mailbox=None, samples=None):
        """``mailbox``: None = the context's default protocol, True/False = this operation's."""
        stream = stream or torch.cuda.current_stream(self.device)
        tokens = max(out.shape[0] for out in outs)
        ctas = self.pick_combine_ctas(tokens, slot.capacity) if ctas is None else ctas
        n = len(self.local_ranks)
        self.engine.combine(list(partials), list(outs), slot.offsets, [slot.capacity] * n, [slot.tokens] * n,
                            identity, ctas, stream.cuda_stream, profile, -1 if mailbox is None else int(bool(mailbox)),
                            samples)
        self.launches += 1

    def scale_rows(self, hidden, local_ids, weights, valid_count, factors, partial, stream=None):
        stream = stream or torch.cuda.current_stream(self.device)
        self.engine.scale_rows(hidden, local_ids, weights, valid_count, factors, partial, stream.cuda_stream)
        self.launches += 1

    def status(self, local: int = 0):
        return self.engine.status(local)
