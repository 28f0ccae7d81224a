"""A whole EP group on ONE GPU: every rank's heap lives on the same device and
each dispatch/combine is a single cooperative launch whose ``blockIdx.y``
selects the rank.

Kernels of different ranks wait on one another, so they may never run as
separate launches on one GPU (nothing guarantees co-residency); one launch
carrying all ranks does. The device code is byte-for-byte the production code:
"peer" pointers simply resolve to the same GPU. This is how the multi-rank
protocol is validated on a single-GPU machine, and how the reference's
"CPU plays the peer" tests (tests/test_host_sm_native_cuda.py:176-186) are
replaced when every rank should really execute.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..config import Config
from .core import Slot, TransportCore


@dataclass(repr=False)
class EmulatedBatch:
    hidden: torch.Tensor
    local_ids: torch.Tensor
    weights: torch.Tensor
    inverse: torch.Tensor
    valid_count: torch.Tensor
    partial: torch.Tensor


class EmulatedGroup:
    def __init__(self, world_size: int, expert_to_rank, config: Config, device=0):
        from .. import native as native_loader
        self.native = native_loader.load()
        if not 1 <= world_size <= self.native.MAX_EMULATED_RANKS:
            raise ValueError(f"an emulated group has between 1 and {self.native.MAX_EMULATED_RANKS} ranks")
        if not config.device_transport:
            raise ValueError("the emulated group runs the device transport")
        self.world_size = world_size
        self.config = config
        self.device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        self.expert_to_rank = [int(owner) for owner in expert_to_rank]
        self._heap_bytes = config.heap_bytes(world_size)
        with torch.cuda.device(self.device):
            self._bases = [self.native.heap_allocate(self._heap_bytes) for _ in range(world_size)]
            self.core = TransportCore(self.native, world=world_size, local_ranks=list(range(world_size)),
                                      heaps=[self._bases] * world_size, heap_bytes=self._heap_bytes, config=config,
                                      expert_to_rank=self.expert_to_rank, device=self.device)
        self._closed = False

    def create_slot(self, capacity: Optional[int] = None, tokens: Optional[int] = None) -> Slot:
        capacity = self.world_size * self.config.max_tokens_per_rank if capacity is None else capacity
        tokens = self.config.max_tokens_per_rank if tokens is None else tokens
        with torch.cuda.device(self.device):
            return self.core.create_slot(capacity, tokens)

    def dispatch(self, slot: Slot, xs, ids, weights, capacities=None, *, ctas=None, identity=0, stream=None):
        capacities = [slot.capacity] * self.world_size if capacities is None else list(capacities)
        with torch.cuda.device(self.device):
            if ctas is None:
                ctas = self.core.pick_ctas(max(x.shape[0] for x in xs))
            self.core.dispatch(slot, xs, ids, weights, capacities, identity=identity, ctas=ctas, stream=stream)
        return [EmulatedBatch(v.hidden[:c], v.local_ids[:c], v.weights[:c], v.inverse[:c], v.count, v.partial[:c])
                for v, c in zip(slot.views, capacities)]

    def combine(self, slot: Slot, partials, token_counts, *, outs=None, ctas=None, identity=0, stream=None,
                mailbox=None):
        with torch.cuda.device(self.device):
            if outs is None:
                outs = [torch.empty((n, self.config.hidden_size), dtype=torch.bfloat16, device=self.device)
                        for n in token_counts]
            if ctas is None:
                ctas = self.core.pick_combine_ctas(max(token_counts), slot.capacity)
            self.core.combine(slot, partials, outs, identity=identity, ctas=ctas, stream=stream, mailbox=mailbox)
        return outs

    def scale_rows(self, batch: EmulatedBatch, factors=None, out=None, stream=None):
        out = batch.partial if out is None else out
        with torch.cuda.device(self.device):
            self.core.scale_rows(batch.hidden, batch.local_ids, batch.weights, batch.valid_count, factors, out, stream)
        return out

    def status(self) -> List[tuple]:
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            return [self.core.status(i) for i in range(self.world_size)]

    def check_guards(self) -> None:
        """Diagnostics: raise if a store landed in the guard band around any live slot."""
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            self.core.check_guards()

    def close(self):
        if self._closed:
            return
        self._closed = True
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            self.core = None
            for base in self._bases:
                self.native.heap_release(base)
        self._bases = []

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        # On an exception the heaps stay mapped until the process ends: whoever formats
        # the error may still print tensors that are views of them.
        if exc_type is None:
            self.close()
        return False
