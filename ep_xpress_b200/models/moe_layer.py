"""A full expert-parallel MoE layer: dispatch -> grouped SwiGLU experts -> combine.

The reference leaves the experts to its serving framework and only adapts that framework's
fused-experts call to the device-resident row count
(ep_xpress/adapters/sglang_valid.py:233-255, ``fused_experts_valid_count``); here the layer is
part of the library, with the same contract: rows at or above ``valid_count`` and slots with
id -1 cost nothing and contribute nothing.
"""

from __future__ import annotations

import torch

from ..ops.moe import GroupedSwiGLU


class SwiGLUMoELayer:
    """Routed experts of one MoE layer, sharded over the ranks of an EP context.

    ``w13``/``w2`` hold THIS rank's experts in the order of their local ids
    (order of appearance in ``expert_to_rank``), K-major as documented in
    :mod:`ep_xpress_b200.ops.moe`.
    """

    def __init__(self, context, w13, w2, *, recv_capacity=None, local_tokens=None, max_local_pairs=None,
                 pair_ctas=True):
        cfg = context.config
        self.context = context
        capacity = context.world_size * cfg.max_tokens_per_rank if recv_capacity is None else recv_capacity
        tokens = cfg.max_tokens_per_rank if local_tokens is None else local_tokens
        self.workspace = context.create_workspace(capacity, tokens)
        self.experts = GroupedSwiGLU(w13, w2, max_rows=capacity, topk=cfg.topk, max_local_pairs=max_local_pairs,
                                     pair_ctas=pair_ctas)
        self.kernel_launches_per_forward = 2 + self.experts.kernel_launches_per_forward

    def forward(self, x, topk_ids, topk_weights, *, stream=None, timing=None):
        ep = self.context
        stream = stream or torch.cuda.current_stream(ep.device)
        marks = [] if timing is not None else None
        if marks is not None:
            marks.append(_mark(stream))
        batch = ep.dispatch_on_stream(x, topk_ids, topk_weights, stream=stream, workspace=self.workspace)
        if marks is not None:
            marks.append(_mark(stream))
        partial = self.experts(batch.hidden, batch.local_ids, batch.weights, batch.valid_count,
                               out=ep.partial_buffer(batch.handle), stream=stream)
        if marks is not None:
            marks.append(_mark(stream))
        out = ep.combine_on_stream(partial, batch.handle, stream=stream)
        if marks is not None:
            marks.append(_mark(stream))
            timing.append(marks)
        return out, batch.valid_count

    __call__ = forward


def _mark(stream):
    event = torch.cuda.Event(enable_timing=True)
    event.record(stream)
    return event
