"""Public API types and the ``Context`` factory.

``Context(nccl_comm=..., expert_to_rank=..., config=...)`` returns the transport
implementation selected by ``config.transport`` (factory in ``__new__`` like the
reference, ep_xpress/context.py:113-120):

* ``"nvlink"`` / ``"host_sm"`` -> :class:`ep_xpress_b200.parallel.nvlink.NVLinkContext`
  (fused sm_100a kernels over peer-mapped HBM);
* ``"host_ce"`` -> :class:`ep_xpress_b200.parallel.host_ce.HostCEContext`
  (host-staged rings; the CPU-visible oracle path);
* ``internode_transport="gin"`` -> not available on a single NVLink domain.

All ranks construct contexts and submit dispatch/combine in the same order;
ranks with zero tokens still participate. A healthy ``close()`` is collective
and must precede destroying the caller's process group. After a failure the
context is poisoned: restart the workers.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .config import Config

ERROR_TEXT = {
    1: "invalid route, inverse map or expert placement",
    2: "receive capacity exceeded",
    3: "timed out waiting for a peer",
    4: "a peer aborted the operation",
    5: "operation identity (tag or handle) mismatch between ranks",
    6: "operation epochs are exhausted (2^31 operations ran on this context): re-create it",
}


@dataclass
class RouteHandle:
    """Inverse route of ONE dispatch; consumable by exactly one combine.

    ``received_count`` is the allocated row count (a capacity); the exact count
    stays on the GPU in ``DispatchBatch.valid_count``.
    """
    _context_id: str
    operation: int
    _plan: object = field(repr=False)
    local_token_count: int
    received_count: int
    tag: object = None
    _consumed: bool = field(default=False, repr=False)

    @property
    def inverse_map(self):
        """Device int64 [capacity, 2] (source rank, source token); rows below valid_count are meaningful."""
        return getattr(self._plan, "inverse", None)

    @property
    def active_channels(self):
        """Launch width chosen at dispatch and reused by combine (None for host_ce)."""
        return getattr(self._plan, "active_channels", None)


@dataclass
class DispatchBatch:
    """Expert inputs of this rank plus the handle that routes results back.

    Device transports return tensors padded to the receive capacity and a CUDA
    ``int32[1]`` ``valid_count``; rows at or above it have ids -1, zero weights
    and zero activations. ``weights`` keeps the weight of every active slot,
    also of experts living on other ranks: mask with ``local_ids >= 0``.
    The tensors are borrowed views of the operation's slot.
    """
    hidden: torch.Tensor
    local_ids: torch.Tensor
    weights: torch.Tensor
    handle: RouteHandle
    valid_count: object


class Pending:
    """Completion ticket of an asynchronous operation."""

    def __init__(self, context, value, completed, workspace=None, tensors=()):
        self._context = context
        self._value = value
        self._completed = completed
        self._workspace = workspace
        self._generation = workspace._generation if workspace is not None else None
        self._tensors = tensors
        self._stats = {}

    def _check_workspace(self):
        if self._workspace is not None and self._generation != self._workspace._generation:
            raise RuntimeError("this ticket has expired: its workspace was reused by a later dispatch")

    def wait(self, stream=None, timeout=None):
        """Make ``stream`` (default: current) wait for the operation; never blocks the CPU."""
        if timeout is not None:
            raise ValueError("device tickets never block the host; timeout is not supported")
        self._check_workspace()
        context = self._context
        with torch.cuda.device(context.device):
            consumer = stream or torch.cuda.current_stream(context.device)
            if consumer.device != context.device:
                raise ValueError("completion stream must belong to the context device")
            consumer.wait_event(self._completed)
            for tensor in self._tensors:
                tensor.record_stream(consumer)
        context._ticket_waited(self, consumer)
        return self._value

    @property
    def done(self):
        self._check_workspace()
        return self._completed.query()

    @property
    def metrics(self):
        return dict(self._stats)


class Context:
    """One long-lived expert-parallel group; one device per process."""

    def __new__(cls, nccl_comm=None, expert_to_rank=None, config=None, device=None, shared_directory=None):
        if cls is Context:
            if not isinstance(config, Config):
                raise TypeError("config must be an ep_xpress_b200.Config")
            if config.internode_transport == "gin":
                from .parallel.multinode import MultiNodeContext
                return object.__new__(MultiNodeContext)
            if config.device_transport:
                from .parallel.nvlink import NVLinkContext
                return object.__new__(NVLinkContext)
            from .parallel.host_ce import HostCEContext
            return object.__new__(HostCEContext)
        return object.__new__(cls)

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        self.close()
        return False

    def check(self):
        """Explicit synchronisation and sticky-error boundary."""
        return self.check_errors()
