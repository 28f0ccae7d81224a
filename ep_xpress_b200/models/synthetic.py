"""The communication-only MoE layer: dispatch -> identity-times-weight expert -> combine.

This is the "model" the reference validates and benchmarks its transports
with (benchmarks/replay.py:67-85, benchmarks/communication.py:154-203): the
expert multiplies every received row by the routing weights of the experts that
live on the rank, so the combined output equals ``x * sum(weights)`` up to the
BF16 rounding steps of the rank-order combine.
"""

from __future__ import annotations

import torch

from ..ops import scale_rows


class IdentityMoELayer:
    def __init__(self, context, *, factors=None, recv_capacity=None, local_tokens=None, use_workspace=True):
        self.context = context
        self.factors = factors
        self.workspace = None
        if use_workspace:
            cfg = context.config
            capacity = context.world_size * cfg.max_tokens_per_rank if recv_capacity is None else recv_capacity
            tokens = cfg.max_tokens_per_rank if local_tokens is None else local_tokens
            self.workspace = context.create_workspace(capacity, tokens)
        self.kernel_launches = 0

    def forward(self, x, topk_ids, topk_weights, *, stream=None, tag=None, timing=None):
        """One layer on ``stream`` (default: current). ``timing`` collects per-phase CUDA events."""
        ep = self.context
        stream = stream or torch.cuda.current_stream(ep.device)
        marks = []
        if timing is not None:
            marks.append(_mark(stream))
        batch = ep.dispatch_on_stream(x, topk_ids, topk_weights, tag=tag, stream=stream, workspace=self.workspace,
                                      recv_capacity=None if self.workspace is not None else None)
        if timing is not None:
            marks.append(_mark(stream))
        partial = scale_rows(ep, batch, self.factors, stream=stream)
        if timing is not None:
            marks.append(_mark(stream))
        out = ep.combine_on_stream(partial, batch.handle, tag=tag, stream=stream)
        if timing is not None:
            marks.append(_mark(stream))
            timing.append(marks)
        self.kernel_launches += 3
        return out, batch.valid_count

    __call__ = forward


def _mark(stream):
    event = torch.cuda.Event(enable_timing=True)
    event.record(stream)
    return event
