"""Per-layer dispatcher an inference engine's MoE layer calls.

Behaviour of the reference's ``HostEPDispatcher`` (ep_xpress/adapters/sglang.py:91-340)
without importing any framework: one ``Context`` is shared by every layer that uses the same
(group, device, config, placement); each layer keeps a small FIFO cache of decode workspaces
keyed by (receive capacity, local tokens); a layer has at most one operation outstanding;
the receive capacity is the scheduler-known sum of token counts; the launch width follows
``select_active_channels``; the DEVICE ``valid_count`` travels to the expert runner and is
never converted to a host integer.
"""

from __future__ import annotations

import logging
from collections import OrderedDict
from dataclasses import dataclass

from .guards import receive_capacity_from_scheduler, select_active_channels

log = logging.getLogger(__name__)
_contexts = {}
_WORKSPACES_PER_LAYER = 4


@dataclass
class DispatchOutput:
    """What the expert runner receives. ``valid_count`` stays on the device."""
    hidden_states: object
    local_expert_ids: object
    weights: object
    valid_count: object
    handle: object


def _context_key(group_key, device, config, placement):
    return (group_key, str(device), config, tuple(placement))


def shared_context(comm, placement, config, *, group_key=None, factory=None):
    """One context per (group, device, config, placement), created on first use."""
    key = _context_key(group_key if group_key is not None else id(comm), getattr(comm, "device", "cpu"), config,
                       placement)
    if key not in _contexts:
        if factory is None:
            from ..context import Context
            factory = Context
        _contexts[key] = factory(comm, list(placement), config)
        log.info("EP context created: world=%s transport=%s channels=%s", getattr(comm, "world_size", "?"),
                 config.transport, getattr(_contexts[key], "effective_channels", None))
    return _contexts[key]


def prepare_graph_capture():
    for context in _contexts.values():
        if hasattr(context, "prepare_graph_capture"):
            context.prepare_graph_capture()


def prepare_graph_replay(stream=None):
    for context in _contexts.values():
        if hasattr(context, "prepare_graph_replay"):
            context.prepare_graph_replay(stream)


def close_contexts():
    while _contexts:
        _, context = _contexts.popitem()
        context.close()


class EPDispatcher:
    def __init__(self, comm, placement, config, *, layer_id, group_key=None, context_factory=None,
                 enable_cuda_graph=False, channel_policy=None):
        self.layer_id = layer_id
        self.config = config
        self.channel_policy = dict(channel_policy or {})     # see adapters.env.channel_policy_from_env
        self.context = shared_context(comm, placement, config, group_key=group_key, factory=context_factory)
        if enable_cuda_graph and not getattr(self.context, "_graph_enabled", False):
            self.context.enable_cuda_graph()
        self._workspaces = OrderedDict()
        self._outstanding = None

    def _workspace(self, capacity, tokens):
        key = (capacity, tokens)
        if key in self._workspaces:
            self._workspaces.move_to_end(key)
            return self._workspaces[key]
        if len(self._workspaces) >= _WORKSPACES_PER_LAYER:
            _, oldest = self._workspaces.popitem(last=False)
            release = getattr(self.context, "release_workspace", None)
            if release is not None:
                release(oldest)
        self._workspaces[key] = self.context.create_workspace(capacity, tokens)
        return self._workspaces[key]

    def dispatch(self, hidden_states, topk_ids, topk_weights, *, token_counts=None, is_decode, stream=None,
                 recv_capacity=None):
        """``token_counts``: scheduled tokens of EVERY rank of the group (host integers), or
        ``recv_capacity``: their sum where the scheduler already publishes it (a padded sum is fine:
        it only has to bound the rows this rank can receive and be the same on every rank)."""
        if self._outstanding is not None:
            raise RuntimeError(f"layer {self.layer_id} already has an operation outstanding; combine it first")
        cfg = self.config
        tokens = hidden_states.shape[0]
        if (token_counts is None) == (recv_capacity is None):
            raise ValueError("pass either token_counts or recv_capacity")
        if recv_capacity is None:
            capacity = receive_capacity_from_scheduler(token_counts, cfg.max_tokens_per_rank)
        else:
            capacity = int(recv_capacity)
            world = getattr(self.context, "world_size", None)
            if capacity < 0 or (world is not None and capacity > world * cfg.max_tokens_per_rank):
                raise ValueError("recv_capacity must lie within [0, world_size * max_tokens_per_rank]")
        small_decode = is_decode and tokens <= max(cfg.decode_max_tokens, 0)
        channels = select_active_channels(tokens, self.context.effective_channels, is_decode=is_decode,
                                          **self.channel_policy)
        kwargs = dict(stream=stream, recv_capacity=capacity, active_channels=channels, tag=("layer", self.layer_id))
        if is_decode or small_decode:
            kwargs["workspace"] = self._workspace(capacity, tokens)
        batch = self.context.dispatch_on_stream(hidden_states, topk_ids, topk_weights, **kwargs)
        self._outstanding = batch.handle
        return DispatchOutput(batch.hidden, batch.local_ids, batch.weights, batch.valid_count, batch.handle)

    def combine(self, partial, *, stream=None):
        if self._outstanding is None:
            raise RuntimeError(f"layer {self.layer_id} has no dispatched operation to combine")
        handle, self._outstanding = self._outstanding, None
        return self.context.combine_on_stream(partial, handle, tag=("layer", self.layer_id), stream=stream)
