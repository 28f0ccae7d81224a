"""Baseline, never the product: dispatch/combine as two ``all_to_all_single`` calls.

This is what an application does without an EP library: deduplicate per
destination rank with tensor ops, exchange per-rank row counts, read them back to
the host (the split sizes of ``all_to_all_single`` are host integers), move the
rows, and on the way back sum the returned partial rows per token. It is timed by
``benchmarks/communication.py --nccl-reference`` on the same shapes as the fused
kernels. The reference's own optional NCCL comparison uses all-gather /
reduce-scatter (benchmarks/communication.py:233-234); all-to-all moves fewer bytes
and is the fairer baseline.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


class NCCLAllToAllBaseline:
    def __init__(self, expert_to_rank, world_size, group=None, device=None):
        self.group = group
        self.world = world_size
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.owner = torch.tensor(list(expert_to_rank), dtype=torch.int64, device=self.device)

    def dispatch(self, x, topk_ids, topk_weights):
        world = self.world
        active = topk_ids >= 0
        dest = self.owner[topk_ids.clamp(min=0).to(torch.int64)]
        hit = torch.zeros((x.shape[0], world), dtype=torch.int32, device=x.device)
        hit.scatter_add_(1, dest, active.to(torch.int32))
        hit = hit > 0                                            # one row per (token, rank)
        pairs = hit.t().nonzero()                                # sorted by destination, then token
        send_counts = hit.sum(dim=0).to(torch.int64)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        in_splits, out_splits = send_counts.tolist(), recv_counts.tolist()       # host sync
        tokens = pairs[:, 1]
        rows = x[tokens]
        recv = torch.empty((sum(out_splits), x.shape[1]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(recv, rows, out_splits, in_splits, group=self.group)
        meta = torch.cat([topk_ids.to(torch.float32), topk_weights.to(torch.float32)], dim=1)[tokens]
        recv_meta = torch.empty((sum(out_splits), meta.shape[1]), dtype=meta.dtype, device=x.device)
        dist.all_to_all_single(recv_meta, meta, out_splits, in_splits, group=self.group)
        state = (tokens, in_splits, out_splits, x.shape[0])
        return recv, recv_meta, state

    def combine(self, partial, state):
        tokens, in_splits, out_splits, count = state
        back = torch.empty((sum(in_splits), partial.shape[1]), dtype=partial.dtype, device=partial.device)
        dist.all_to_all_single(back, partial, in_splits, out_splits, group=self.group)
        out = torch.zeros((count, partial.shape[1]), dtype=torch.float32, device=partial.device)
        out.index_add_(0, tokens, back.to(torch.float32))
        return out.to(torch.bfloat16)
