"""The NVLink transport: one rank of an EP group on one B200.

Lifecycle and API follow the reference's device transport
(ep_xpress/host_sm.py:274-1234): construct collectively, dispatch/combine in
the same order on every rank, ``check()`` at explicit boundaries, ``close()``
collectively. The differences are physical: payloads are stored into and
loaded from peer HBM by the fused sm_100a kernels, the only per-operation host
work is argument checking and one cooperative launch, and generation counters
always live on the device, so eager and CUDA-graph execution share one code
path (the reference switches to device epochs in ``enable_cuda_graph``,
host_sm.py:809-830).
"""

from __future__ import annotations

import contextlib
import hashlib
import json
import socket
import threading
import uuid
from dataclasses import asdict, dataclass

import torch

from ..comm import ControlPlane
from ..config import Config
from ..context import ERROR_TEXT, Context, DispatchBatch, Pending, RouteHandle
from .core import Slot, TransportCore

_MAX_EPOCHS = (1 << 31) - 1


def operation_identity(phase, tag, dispatch_operation=None) -> int:
    """64-bit identity of (phase, tag, dispatch number); only used with diagnostics."""
    text = json.dumps([phase, tag, dispatch_operation], sort_keys=True, separators=(",", ":"))
    return int.from_bytes(hashlib.blake2b(text.encode(), digest_size=8).digest(), "little")


@dataclass
class _DeviceRoute:
    slot: Slot
    inverse: torch.Tensor
    count: torch.Tensor
    active_channels: int
    ctas: int
    expected_ranks: torch.Tensor
    dest_rows: torch.Tensor
    workspace: object
    capacity: int
    fused_combine: bool
    combine_ctas: int = 0


class Workspace:
    """Explicitly retained storage of one (capacity, local tokens, fused) shape.

    Batches, outputs and tickets are borrowed until this workspace's next
    dispatch (contract of ep_xpress/host_sm.py:128-199).
    """

    def __init__(self, context, recv_capacity, local_tokens, fused_combine):
        self._context_id = context._id
        self.recv_capacity = recv_capacity
        self.local_tokens = local_tokens
        self.fused_combine = fused_combine
        self._slot = context._core.create_slot(max(recv_capacity, 1), max(local_tokens, 1))
        views = self._slot.views[0]
        self.hidden = views.hidden[:recv_capacity]
        self.local_ids = views.local_ids[:recv_capacity]
        self.weights = views.weights[:recv_capacity]
        self.inverse = views.inverse[:recv_capacity]
        self.partial = views.partial[:recv_capacity]
        self.count = views.count
        self.output = views.output[:local_tokens]
        self.expected_ranks = views.mask[:local_tokens]
        self.dest_rows = views.dest_rows[:local_tokens]
        self._generation = 0
        self._busy = False
        self._consumers = []

    def _acquire(self, execution, *, capturing=False):
        if not capturing:
            for consumer in self._consumers:
                if consumer != execution:
                    execution.wait_stream(consumer)
        self._consumers = []
        self._generation += 1
        self._busy = True

    def _combined(self, consumer, *, capturing=False):
        self._busy = False
        if not capturing and consumer not in self._consumers:
            self._consumers.append(consumer)


class NVLinkContext(Context):
    """See :class:`ep_xpress_b200.Context`."""

    def __init__(self, nccl_comm, expert_to_rank, config, device=None, shared_directory=None):
        if not isinstance(nccl_comm, ControlPlane) or not hasattr(nccl_comm, "all_gather_object"):
            raise TypeError("nccl_comm must be an NCCLCommHandle (see get_nccl_comm_handle)")
        if not isinstance(config, Config) or not config.device_transport:
            raise TypeError("config must select a device transport")
        self.config = config
        inert = config.inert_fields()
        if inert:
            import warnings
            warnings.warn("these Config fields have no effect on the NVLink transport: " + ", ".join(inert),
                          stacklevel=3)
        self._comm = nccl_comm
        self.rank, self.world_size = nccl_comm.rank, nccl_comm.world_size
        if not 1 <= self.world_size <= 63:
            raise ValueError("the EP group must have between 1 and 63 ranks")
        owners = [int(owner) for owner in (expert_to_rank.tolist() if isinstance(expert_to_rank, torch.Tensor)
                                           else expert_to_rank)]
        if not owners or any(not 0 <= owner < self.world_size for owner in owners):
            raise ValueError("expert_to_rank must map every expert to a rank of the group")
        if config.topk > len(owners):
            raise ValueError("topk exceeds the number of experts")
        if self.world_size * config.max_tokens_per_rank > (1 << 31) - 1:
            raise ValueError("world_size * max_tokens_per_rank must fit int32")
        self.expert_to_rank = owners
        comm_device = torch.device(nccl_comm.device)
        chosen = comm_device if device is None else torch.device(device)
        if chosen.type == "cuda" and chosen.index is None:
            chosen = torch.device("cuda", torch.cuda.current_device())
        if chosen != comm_device:
            raise ValueError("the context and its NCCL communicator must use the same CUDA device")
        self.device = chosen
        self._id = uuid.uuid4().hex
        self._lock = threading.RLock()
        self._failed = None
        self._closed = False
        self._counter = 0
        self._pending = 0
        self._graph_enabled = False
        self._capture_ready = False
        self._last_stream = None
        self._pool = []
        self._workspaces = []
        self._profile = None
        self._max_receive_capacity = self.world_size * config.max_tokens_per_rank
        self._heap_base = None
        self._peer_bases = []
        self._bootstrap()

    # ------------------------------------------------------------------ bootstrap
    def _bootstrap(self):
        from .. import native as native_loader
        native = native_loader.load()
        comm, config = self._comm, self.config
        signature = {"config": asdict(config), "placement": tuple(self.expert_to_rank),
                     "build": native_loader.build_identity(), "world": self.world_size}
        gathered = comm.all_gather_object({"signature": signature, "host": socket.gethostname()})
        if any(entry["signature"] != signature for entry in gathered):
            raise ValueError("EP ranks were constructed with a different configuration, placement or native build")
        heap_bytes = config.heap_bytes(self.world_size)
        if heap_bytes > config.gpu_pool_budget_bytes:
            raise ValueError(f"the negotiated peer-mapped heap ({heap_bytes} bytes) exceeds gpu_pool_budget_bytes")
        error, handle = None, None
        with torch.cuda.device(self.device):
            try:
                self._heap_base = native.heap_allocate(heap_bytes)
                handle = native.heap_export(self._heap_base)
            except Exception as exc:  # reported collectively below
                error = repr(exc)
            exported = comm.all_gather_object((handle, error))
            failures = [f"rank {r}: {e}" for r, (_, e) in enumerate(exported) if e]
            if failures:
                self._release_resources()
                raise RuntimeError("peer heap allocation failed: " + "; ".join(failures))
            bases = []
            try:
                for peer, (peer_handle, _) in enumerate(exported):
                    if peer == self.rank:
                        bases.append(self._heap_base)
                    else:
                        base = native.heap_open(peer_handle, heap_bytes)
                        self._peer_bases.append(base)
                        bases.append(base)
                self._core = TransportCore(native, world=self.world_size, local_ranks=[self.rank], heaps=[bases],
                                           heap_bytes=heap_bytes, config=config,
                                           expert_to_rank=self.expert_to_rank, device=self.device)
                local_max = self._core.max_ctas
            except Exception as exc:
                error, local_max = repr(exc), 0
            negotiated = comm.all_gather_object((local_max, error))
            failures = [f"rank {r}: {e}" for r, (_, e) in enumerate(negotiated) if e]
            if failures:
                self._release_resources()
                raise RuntimeError("peer heap mapping failed: " + "; ".join(failures))
            self._core.max_ctas = min(width for width, _ in negotiated)
            self._negotiated_ctas = self._core.max_ctas
            self.effective_channels = min(config.channels, 32)
            self._work_stream = torch.cuda.Stream(self.device)
            comm.barrier()

    # ------------------------------------------------------------------ health
    def _check_usable(self):
        if self._closed:
            raise RuntimeError("EP context is closed")
        if self._failed is not None:
            raise RuntimeError("EP context is in a failed state") from self._failed

    def _abort(self, error):
        if self._failed is None:
            self._failed = error

    def check_errors(self):
        """Synchronise this context's streams and raise the sticky device error, if any."""
        with self._lock, torch.cuda.device(self.device):
            self._check_usable()
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("check() cannot run during CUDA Graph capture")
            self._work_stream.synchronize()
            if self._last_stream is not None:
                self._last_stream.synchronize()
            status, detail, _, _ = self._core.status(0)
            if status:
                text = ERROR_TEXT.get(status, f"unknown device status {status}")
                error = RuntimeError(f"{self.config.transport}: {text} (detail 0x{detail:016x})")
                self._abort(error)
                raise error
            if self.config.diagnostics:
                try:
                    self._core.check_guards()
                except RuntimeError as error:
                    self._abort(error)
                    raise

    def stats(self):
        """Counters of this context (launches, epochs, heap use); synchronises the device."""
        with self._lock, torch.cuda.device(self.device):
            status, detail, dispatch_epoch, combine_epoch = self._core.status(0)
            return {"status": status, "detail": detail, "dispatch_epoch": dispatch_epoch,
                    "combine_epoch": combine_epoch, "launches": self._core.launches,
                    "heap_free_bytes": self._core._allocators[0].free_bytes,
                    "max_ctas": self._core.max_ctas, "effective_channels": self.effective_channels}

    # ------------------------------------------------------------------ graphs
    def set_tuning(self, *, items_per_cta=None, max_ctas=None):
        """Launch-width policy: a CTA is launched per ``items_per_cta`` (token, 2 KiB row segment)
        work items, at most ``max_ctas`` (never above the width negotiated at bootstrap). Call it
        between operations, before graph capture; every rank may choose its own values."""
        with self._lock:
            if items_per_cta is not None:
                if int(items_per_cta) < 1:
                    raise ValueError("items_per_cta must be positive")
                self._core.items_per_cta = int(items_per_cta)
            if max_ctas is not None:
                if not 1 <= int(max_ctas) <= self._negotiated_ctas:
                    raise ValueError(f"max_ctas must be within 1..{self._negotiated_ctas}")
                self._core.max_ctas = int(max_ctas)

    def enable_cuda_graph(self):
        """Allow capture of direct-stream operations. Call on every rank, outside capture."""
        with self._lock:
            self._check_usable()
            if self.config.diagnostics:
                raise RuntimeError("CUDA Graph mode requires diagnostics to be disabled")
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("enable_cuda_graph must be called outside capture")
            self._graph_enabled = True

    def prepare_graph_capture(self):
        """Drain this context on the host and arm capture."""
        with self._lock, torch.cuda.device(self.device):
            self._check_usable()
            if not self._graph_enabled:
                raise RuntimeError("enable_cuda_graph is required before prepare_graph_capture")
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("prepare_graph_capture must be called outside capture")
            self._work_stream.synchronize()
            if self._last_stream is not None:
                self._last_stream.synchronize()
            self._capture_ready = True

    def prepare_graph_replay(self, stream=None):
        """Order ``stream`` after the context's previous stream before a replay (no host sync)."""
        with self._lock, torch.cuda.device(self.device):
            self._check_usable()
            if not self._graph_enabled:
                raise RuntimeError("enable_cuda_graph is required before prepare_graph_replay")
            stream = stream or torch.cuda.current_stream(self.device)
            if self._last_stream is not None and self._last_stream != stream:
                stream.wait_stream(self._last_stream)
            self._last_stream = stream

    def _check_capture(self, *, same_stream):
        """Lifecycle misuse is a caller error: it is raised before anything is enqueued and
        does not poison the context."""
        if not torch.cuda.is_current_stream_capturing():
            return False
        if not (self._graph_enabled and self._capture_ready):
            raise RuntimeError("prepare_graph_capture is required before capturing EP operations")
        if not same_stream:
            raise RuntimeError("CUDA Graph capture requires direct-stream operations")
        return True

    def _begin(self, execution, *, capturing):
        """Serialise this operation after the context's previous one."""
        self._counter += 1
        if self._counter >= _MAX_EPOCHS:
            raise RuntimeError("operation epochs are exhausted; recreate the context")
        if not capturing and self._last_stream is not None and self._last_stream != execution:
            execution.wait_stream(self._last_stream)
        self._last_stream = execution

    # ------------------------------------------------------------------ workspaces
    def create_workspace(self, recv_capacity, local_tokens, *, fused_combine=False):
        with self._lock, torch.cuda.device(self.device):
            self._check_usable()
            self._validate_workspace_shape(recv_capacity, local_tokens, fused_combine)
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("workspaces must be created outside CUDA Graph capture")
            workspace = Workspace(self, recv_capacity, local_tokens, fused_combine)
            self._workspaces.append(workspace)
            return workspace

    def release_workspace(self, workspace):
        """Return a workspace's heap range; its tensors must no longer be in use."""
        with self._lock:
            if not isinstance(workspace, Workspace) or workspace._context_id != self._id:
                raise ValueError("workspace belongs to another context")
            if workspace._busy:
                raise RuntimeError("wait on the previous workspace combine before releasing it")
            self._core.release_slot(workspace._slot)
            if workspace in self._workspaces:
                self._workspaces.remove(workspace)

    def _validate_workspace_shape(self, capacity, local_tokens, fused_combine):
        for name, value, upper in (("recv_capacity", capacity, self._max_receive_capacity),
                                   ("local_tokens", local_tokens, self.config.max_tokens_per_rank)):
            if isinstance(value, bool) or not isinstance(value, int) or not 0 <= value <= upper:
                raise ValueError(f"{name} must be an integer within the configured rank capacity")
        if not isinstance(fused_combine, bool):
            raise ValueError("fused_combine must be a bool")
        if fused_combine and (not self.config.decode_max_tokens or local_tokens > self.config.decode_max_tokens):
            raise ValueError("fused combine requires local tokens within the configured decode mailbox capacity")

    def _acquire_pool_slot(self):
        for slot in self._pool:
            if not slot.busy:
                return slot
        if len(self._pool) < self.config.slots:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("CUDA Graph capture requires a warmed, retained workspace")
            slot = self._core.create_slot(self._max_receive_capacity, self.config.max_tokens_per_rank,
                                          self._work_stream)
            # The reset of the fresh slot runs on the context's stream: whichever stream executes
            # the slot's first dispatch has to wait for it (see `_dispatch`).
            slot.reset_done = torch.cuda.Event()
            slot.reset_done.record(self._work_stream)
            self._pool.append(slot)
            return slot
        raise RuntimeError(f"all {self.config.slots} operation slots hold handles that were not combined yet; "
                           "combine one first, use workspaces, or raise Config.slots")

    # ------------------------------------------------------------------ dispatch
    def _validate_dispatch(self, x, ids, weights):
        """Host-side checks only: shapes, dtypes and devices are checked again by the engine."""
        for name, tensor in (("x", x), ("topk_ids", ids), ("topk_weights", weights)):
            if not isinstance(tensor, torch.Tensor):
                raise ValueError(f"dispatch inputs must be tensors ({name} is {type(tensor).__name__})")
        limit = self.config.max_tokens_per_rank
        if x.ndim != 2 or x.shape[0] > limit:
            raise ValueError(f"x must be [tokens, hidden] within the configured token capacity of {limit}")
        if x.requires_grad or weights.requires_grad:
            raise ValueError("dispatch accepts inference tensors only (requires_grad is set)")

    def dispatch_on_stream(self, x, topk_ids, topk_weights, tag=None, stream=None, recv_capacity=None,
                           active_channels=None, workspace=None, fused_combine=False):
        """Enqueue dispatch on the caller's stream and return its batch (no ticket, no event)."""
        return self._dispatch(x, topk_ids, topk_weights, tag, stream, recv_capacity, active_channels, workspace,
                              fused_combine, same_stream=True)

    def dispatch_async(self, x, topk_ids, topk_weights, tag=None, stream=None, recv_capacity=None,
                       active_channels=None, workspace=None, fused_combine=False):
        """Enqueue dispatch on the context's stream; ``.wait(stream)`` the returned ticket."""
        return self._dispatch(x, topk_ids, topk_weights, tag, stream, recv_capacity, active_channels, workspace,
                              fused_combine, same_stream=False)

    def _dispatch(self, x, topk_ids, topk_weights, tag, stream, recv_capacity, active_channels, workspace,
                  fused_combine, *, same_stream):
        with self._lock, torch.cuda.device(self.device):
            self._check_usable()
            self._validate_dispatch(x, topk_ids, topk_weights)
            capacity = ((workspace.recv_capacity if isinstance(workspace, Workspace)
                         else self._max_receive_capacity) if recv_capacity is None else recv_capacity)
            self._validate_workspace_shape(capacity, x.shape[0], fused_combine)
            if workspace is not None:
                if not isinstance(workspace, Workspace) or workspace._context_id != self._id:
                    raise ValueError("workspace belongs to another context")
                wanted = (capacity, x.shape[0], fused_combine)
                if wanted != (workspace.recv_capacity, workspace.local_tokens, workspace.fused_combine):
                    raise ValueError(f"workspace shape or fused combine mode does not match dispatch: the dispatch "
                                     f"needs (capacity, tokens, fused) = {wanted}")
                if workspace._busy:
                    raise RuntimeError("this workspace still holds a dispatch without its combine: wait on the "
                                       "previous workspace combine before reusing it")
            channels = self.effective_channels if active_channels is None else active_channels
            if isinstance(channels, bool) or not isinstance(channels, int) or \
                    not 1 <= channels <= self.effective_channels:
                raise ValueError("active_channels must be an integer within the allocated channel count")
            if not same_stream and self._pending >= self.config.max_pending_operations:
                raise RuntimeError("too many pending operations; wait on earlier tickets first")
            identity = operation_identity("dispatch", tag) if self.config.diagnostics else 0
            producer = stream or torch.cuda.current_stream(self.device)
            execution = producer if same_stream else self._work_stream
            capturing = self._check_capture(same_stream=same_stream)
            if capturing and (workspace is None or workspace._generation == 0):
                raise RuntimeError("CUDA Graph capture requires a warmed, retained workspace")
            slot = workspace._slot if workspace is not None else self._acquire_pool_slot()
            try:
                self._begin(execution, capturing=capturing)
                if not same_stream:
                    execution.wait_stream(producer)
                if workspace is not None:
                    workspace._acquire(execution, capturing=capturing)
                reset_done = getattr(slot, "reset_done", None)
                if reset_done is not None:
                    execution.wait_event(reset_done)
                    slot.reset_done = None
                ids = topk_ids if topk_ids.is_contiguous() else topk_ids.contiguous()
                weights = topk_weights if topk_weights.is_contiguous() else topk_weights.contiguous()
                if ids.dtype not in (torch.int32, torch.int64):
                    raise ValueError("topk_ids must be int32 or int64")
                if x.data_ptr() % 4:
                    x = x.clone()
                budget = max(1, self._core.max_ctas * channels // self.effective_channels)
                ctas = self._core.pick_ctas(x.shape[0], budget)
                combine_ctas = self._core.pick_combine_ctas(x.shape[0], capacity, budget)
                profile = None if self._profile is None else self._profile.slice_for(
                    "dispatch", self._counter, tag, x.shape[0], capacity, ctas)
                with self._on(execution, stream, same_stream):
                    if not same_stream:
                        for tensor in (x, ids, weights):
                            tensor.record_stream(execution)
                    self._core.dispatch(slot, [x], [ids], [weights], [capacity], identity=identity, ctas=ctas,
                                        stream=execution, profile=profile, samples=self._sample_ring("dispatch"))
            except BaseException as error:
                self._abort(error)
                raise
            slot.busy = True
            slot.generation += 1
            views = slot.views[0]
            if workspace is not None:
                # A workspace has exactly this shape: its views were cut once, at creation
                # (slicing six tensors costs more host time than the rest of the call).
                route = _DeviceRoute(slot, workspace.inverse, views.count, channels, ctas, workspace.expected_ranks,
                                     workspace.dest_rows, workspace, capacity, fused_combine, combine_ctas)
                handle = RouteHandle(self._id, self._counter, route, x.shape[0], capacity, tag)
                batch = DispatchBatch(workspace.hidden, workspace.local_ids, workspace.weights, handle, views.count)
            else:
                route = _DeviceRoute(slot, views.inverse[:capacity], views.count, channels, ctas,
                                     views.mask[:x.shape[0]], views.dest_rows[:x.shape[0]], workspace, capacity,
                                     fused_combine, combine_ctas)
                handle = RouteHandle(self._id, self._counter, route, x.shape[0], capacity, tag)
                batch = DispatchBatch(views.hidden[:capacity], views.local_ids[:capacity], views.weights[:capacity],
                                      handle, views.count)
            if same_stream:
                return batch
            return self._finish(batch, workspace, metrics={"ctas": ctas, "active_channels": channels,
                                                           "recv_capacity": capacity})

    @staticmethod
    def _on(execution, requested, same_stream):
        """Make ``execution`` the current stream for the torch allocations and copies of an
        operation - unless it already is (a direct call on the caller's current stream), where
        entering the context would only cost host time. Inputs are inference tensors and the
        kernels are launched outside autograd, so no grad mode is touched."""
        if same_stream and requested is None:
            return contextlib.nullcontext()
        return torch.cuda.stream(execution)

    def _finish(self, value, workspace=None, tensors=(), metrics=None):
        completed = torch.cuda.Event()
        completed.record(self._work_stream)
        self._pending += 1
        ticket = Pending(self, value, completed, workspace, tensors)
        ticket._stats = dict(metrics or {})
        return ticket

    def _ticket_waited(self, ticket, consumer):
        with self._lock:
            if not getattr(ticket, "_counted", False):
                ticket._counted = True
                self._pending = max(0, self._pending - 1)
            workspace = ticket._workspace
            if workspace is not None and not isinstance(ticket._value, DispatchBatch):
                workspace._combined(consumer)

    def partial_buffer(self, handle):
        """The peer-visible partial plane of ``handle``'s slot, BF16 [capacity, hidden].

        An expert runner that writes its weighted output here lets combine skip
        the local copy into the heap. Borrowed like the batch tensors.
        """
        if not isinstance(handle, RouteHandle) or handle._context_id != self._id:
            raise ValueError("handle belongs to another context")
        return handle._plan.slot.views[0].partial[:handle._plan.capacity]

    # ------------------------------------------------------------------ combine
    def combine_on_stream(self, partial, handle, tag=None, stream=None, weights_applied=True):
        """Enqueue combine on the caller's stream and return the output tensor."""
        return self._combine(partial, handle, tag, stream, weights_applied, same_stream=True)

    def combine_async(self, partial, handle, tag=None, stream=None, weights_applied=True):
        return self._combine(partial, handle, tag, stream, weights_applied, same_stream=False)

    def _combine(self, partial, handle, tag, stream, weights_applied, *, same_stream):
        with self._lock, torch.cuda.device(self.device):
            self._check_usable()
            mine = isinstance(handle, RouteHandle) and handle._context_id == self._id
            if not mine:
                raise ValueError("handle belongs to another context")
            if handle._consumed:
                raise ValueError("handle has already been consumed by combine")
            if weights_applied is not True:
                raise ValueError("combine accepts already-weighted rank partials only")
            if not isinstance(partial, torch.Tensor) or partial.requires_grad:
                raise ValueError("partial must be an inference tensor")
            # Every received row owes its token's owner a result row, so the partial tensor covers
            # the dispatch's whole receive capacity (shape rule of ep_xpress/context.py:380).
            rows_ok = partial.ndim == 2 and partial.shape[0] == handle.received_count
            if not rows_ok or partial.shape[1] != self.config.hidden_size or partial.dtype != torch.bfloat16:
                raise ValueError(f"partial must be BF16 [{handle.received_count}, {self.config.hidden_size}]: one "
                                 "row per row of the dispatch's receive capacity")
            if not same_stream and self._pending >= self.config.max_pending_operations:
                raise RuntimeError("too many pending operations; wait on earlier tickets first")
            route = handle._plan
            workspace = route.workspace
            identity = operation_identity("combine", tag, handle.operation) if self.config.diagnostics else 0
            producer = stream or torch.cuda.current_stream(self.device)
            execution = producer if same_stream else self._work_stream
            capturing = self._check_capture(same_stream=same_stream)
            try:
                self._begin(execution, capturing=capturing)
                if not same_stream:
                    execution.wait_stream(producer)
                with self._on(execution, stream, same_stream):
                    source = partial if partial.is_contiguous() else partial.contiguous()
                    if not same_stream:
                        source.record_stream(execution)
                    if workspace is None:
                        output = torch.empty((handle.local_token_count, self.config.hidden_size),
                                             dtype=torch.bfloat16, device=self.device)
                    else:
                        output = workspace.output
                    profile = None if self._profile is None else self._profile.slice_for(
                        "combine", handle.operation, tag, handle.local_token_count, handle.received_count,
                        route.combine_ctas)
                    # Receive-and-reduce in one pass (the mailbox protocol) is the default wherever it
                    # applies; `fused_combine=True` at dispatch asks for it even when the context's
                    # default is the sequential protocol (Config.combine_streaming="off").
                    self._core.combine(route.slot, [source], [output], identity=identity, ctas=route.combine_ctas,
                                       stream=execution, profile=profile,
                                       mailbox=True if route.fused_combine else None,
                                       samples=self._sample_ring("combine"))
            except BaseException as error:
                self._abort(error)
                raise
            handle._consumed = True
            if workspace is None:
                route.slot.busy = False
            if same_stream:
                if workspace is not None:
                    workspace._combined(execution, capturing=capturing)
                return output
            return self._finish(output, workspace, tensors=() if workspace is not None else (output,),
                                metrics={"ctas": route.combine_ctas, "active_channels": route.active_channels})

    # ------------------------------------------------------------------ profiling
    def start_combine_profile(self, max_operations=1024):
        from ..utils.profile import OperationProfile
        with self._lock:
            self._check_usable()
            if self._profile is not None:
                raise RuntimeError("stop the current profile before starting another")
            self._profile = OperationProfile(self, max_operations)

    def set_combine_profile_label(self, label):
        with self._lock:
            if self._profile is None:
                raise RuntimeError("no profile is running")
            self._profile.label = label

    def stop_combine_profile(self):
        with self._lock:
            if self._profile is None:
                raise RuntimeError("no profile is running")
            profile, self._profile = self._profile, None
            with torch.cuda.device(self.device):
                self._work_stream.synchronize()
                if self._last_stream is not None:
                    self._last_stream.synchronize()
                self._last_profile = profile.finish()
            return self._last_profile

    def read_combine_profile(self):
        """The last completed report; never synchronises and never reads device memory."""
        if self._profile is not None:
            raise RuntimeError("stop the combine profile at a completed boundary before reading it")
        report = getattr(self, "_last_profile", None)
        if report is None:
            raise RuntimeError("no completed profile is available")
        return report

    # ---- decode profile: fixed storage that captured operations keep writing into -----------
    def prepare_decode_profile(self, max_samples_per_channel=1024, *, stage="combine"):
        """Install a bounded sample ring that every operation of ``stage`` records into.

        ``stage`` is "dispatch", "combine" or "layer" (both). Call it before the graphs that
        should be measured are captured (same rule as the reference,
        ep_xpress/host_sm.py:515-545): a captured kernel carries the ring's address. Every
        operation launched afterwards - eager or replayed - records one sample while the profile
        is started: the earliest start and the latest end over its CTAs on the GPU's global
        timer. The ring holds ``max_samples_per_channel`` operations per stage; later ones are
        counted as ``dropped_samples``. Nothing is recorded, and the kernels do not touch the
        ring's rows, between ``stop`` and the next ``start``.
        """
        with self._lock, torch.cuda.device(self.device):
            self._check_usable()
            if stage not in ("dispatch", "combine", "layer"):
                raise ValueError("stage must be dispatch, combine or layer")
            if isinstance(max_samples_per_channel, bool) or not isinstance(max_samples_per_channel, int) \
                    or not 1 <= max_samples_per_channel <= 1 << 20:
                raise ValueError("max_samples_per_channel must be an integer in [1, 2^20]")
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("prepare_decode_profile must be called before graph capture")
            words = self._core.native.SAMPLE_WORDS
            stages = ("dispatch", "combine") if stage == "layer" else (stage,)
            self._decode_profile = {
                "stage": stage, "capacity": max_samples_per_channel, "running": False,
                "rings": {name: torch.zeros((1, 1 + max_samples_per_channel, words), dtype=torch.int64,
                                            device=self.device) for name in stages}}

    def _sample_ring(self, stage):
        state = getattr(self, "_decode_profile", None)
        return None if state is None else state["rings"].get(stage)

    def start_decode_profile(self):
        """Begin recording at a quiescent boundary: synchronises the device, clears the rings and
        maps the next operation of each stage to sample 0."""
        state = getattr(self, "_decode_profile", None)
        if state is None:
            raise RuntimeError("prepare_decode_profile is required before the first capture")
        with self._lock, torch.cuda.device(self.device):
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("start_decode_profile must be called outside capture")
            torch.cuda.synchronize(self.device)
            _, _, dispatch_epoch, combine_epoch = self._core.status(0)
            for name, ring in state["rings"].items():
                ring.zero_()
                ring[0, 1:, 0] = torch.iinfo(torch.int64).max          # earliest start: preset to "never"
                ring[0, 0, 1] = (dispatch_epoch if name == "dispatch" else combine_epoch) + 1
                ring[0, 0, 2] = 1
            torch.cuda.synchronize(self.device)
            state["running"] = True

    def stop_decode_profile(self):
        """Stop recording (synchronises the device) and return the samples of every stage:
        ``{"stages": {name: {"samples": n, "dropped_samples": d, "begin_ns": [...], "elapsed_ns": [...]}}}``,
        one entry per operation since ``start`` in submission order."""
        state = getattr(self, "_decode_profile", None)
        if state is None:
            raise RuntimeError("prepare_decode_profile is required before the first capture")
        if not state["running"]:
            raise RuntimeError("start_decode_profile is required before stop_decode_profile")
        with self._lock, torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            report = {"schema": 2, "stage": state["stage"], "max_samples_per_channel": state["capacity"],
                      "stages": {}}
            for name, ring in state["rings"].items():
                ring[0, 0, 2] = 0
                host = ring[0].cpu()
                rows = host[1:]
                used = int((rows[:, 2] > 0).sum())
                begin, end = rows[:used, 0], rows[:used, 1]
                report["stages"][name] = {"samples": used, "dropped_samples": int(host[0, 0]),
                                          "begin_ns": begin.tolist(), "elapsed_ns": (end - begin).tolist(),
                                          "ctas": rows[:used, 2].tolist()}
            state["running"] = False
        return report

    # ------------------------------------------------------------------ teardown
    def _release_resources(self, *, keep_own_heap=False):
        from .. import native as native_loader
        native = native_loader.load()
        for base in self._peer_bases:
            try:
                native.heap_release(base)
            except Exception:
                pass
        self._peer_bases = []
        if self._heap_base is not None and not keep_own_heap:
            try:
                native.heap_release(self._heap_base)
            except Exception:
                pass
            self._heap_base = None

    def close(self):
        """Collective on healthy contexts: drain, rendezvous, unmap, free.

        After a failure there is no rendezvous (a peer may be gone): peer mappings
        are dropped, but this rank's own heap stays allocated until the process
        exits, because surviving peers may still store flag words into it.
        """
        with self._lock:
            if self._closed:
                return
            self._closed = True
            with torch.cuda.device(self.device):
                torch.cuda.synchronize(self.device)
                healthy = self._failed is None
                if healthy:
                    self._comm.barrier()
                self._pool = []
                self._workspaces = []
                self._core = None
                self._release_resources(keep_own_heap=not healthy)
