"""Expert parallelism across nodes, over the point-to-point path of the borrowed communicator.

Selected by ``Config(transport="host_sm", internode_transport="gin")``, the reference's switch
for its multi-node transport (ep_xpress/multinode.py:90-368). The reference drives NCCL's
device-initiated puts from its own kernels; between nodes the wire is the bottleneck, not the
launch path, so this transport keeps the contract and moves records with grouped
``ncclSend``/``ncclRecv`` on the communicator it borrowed (``ControlPlane.exchange``):

* 2 to 256 ranks (destination sets are per-rank columns, not 64-bit masks);
* one activation row per (token, destination rank); rows arrive ordered by (source rank,
  token); outputs are padded to a CPU-known capacity, ``valid_count`` stays an ``int32[1]``
  tensor on the context device; padding rows have ids -1, zero weights and zero activations;
* ``weights`` of slots whose expert lives on another rank are zero (the multi-node reference
  clears them, ep_xpress/csrc/gin.cu:189);
* combine: ONE FP32 accumulation over all contributing ranks in global rank order, the local
  rank included, and a single rounding (ep_xpress/csrc/gin.cu:226-246); ``combine_rounding=
  "two_step"`` selects the single-node formula instead;
* a combine must carry the tag of its dispatch; handles are bounded by
  ``max_pending_operations`` and may be combined in any rank-consistent order;
* every rank learns the whole count matrix of a dispatch before any payload moves, so an
  invalid route or an undersized capacity anywhere fails the operation on every rank, without
  a hang.

The sizes of the transfers are read back to the host once per dispatch (they are arguments of
the NCCL calls), so these operations cannot be captured into CUDA graphs. On CPU tensors the
same code runs over any ``torch.distributed`` group (``GroupControlPlane``), which is how the
protocol is tested without a second node.
"""

from __future__ import annotations

import os
import socket
import threading
import uuid
from dataclasses import asdict, dataclass
from typing import List

import torch

from ..comm import ControlPlane
from ..config import Config
from ..context import ERROR_TEXT, Context, DispatchBatch, RouteHandle
from .host_ce import CompletedTicket


def node_identity() -> str:
    """Same for all processes of one host, containers included (the kernel's boot id)."""
    override = os.environ.get("EPX_NODE_ID")
    if override:
        return override
    try:
        with open("/proc/sys/kernel/random/boot_id") as handle:
            return handle.read().strip()
    except OSError:
        return socket.gethostname()


class MultiNodeWorkspace:
    """Retained tensors of one (capacity, local tokens) shape; borrowed until its next dispatch."""

    def __init__(self, context, recv_capacity, local_tokens, fused_combine):
        cfg, device = context.config, context.device
        self.context_id = context._id
        self.recv_capacity, self.local_tokens, self.fused_combine = recv_capacity, local_tokens, fused_combine
        self.hidden = torch.zeros((recv_capacity, cfg.hidden_size), dtype=torch.bfloat16, device=device)
        self.local_ids = torch.full((recv_capacity, cfg.topk), -1, dtype=torch.int64, device=device)
        self.weights = torch.zeros((recv_capacity, cfg.topk), dtype=torch.float32, device=device)
        self.inverse = torch.full((recv_capacity, 2), -1, dtype=torch.int64, device=device)
        self.count = torch.zeros(1, dtype=torch.int32, device=device)
        self.output = torch.zeros((local_tokens, cfg.hidden_size), dtype=torch.bfloat16, device=device)
        self.generation = 0
        self.busy = False


@dataclass
class _Route:
    workspace: MultiNodeWorkspace
    generation: int
    sent_tokens: List[torch.Tensor]      # per destination rank: indices of my tokens, ascending
    received: List[int]                  # rows every source rank sent me
    inverse: torch.Tensor
    count: torch.Tensor
    active_channels: int


class MultiNodeContext(Context):
    def __init__(self, nccl_comm, expert_to_rank, config, device=None, shared_directory=None):
        if not isinstance(nccl_comm, ControlPlane):
            raise TypeError("Context requires an upper-layer NCCLCommHandle")
        if not isinstance(config, Config) or config.internode_transport != "gin":
            raise TypeError("config must select the multi-node transport")
        self._comm, self.config = nccl_comm, config
        self.rank, self.world_size = nccl_comm.rank, nccl_comm.world_size
        if not 2 <= self.world_size <= 256:
            raise ValueError("GIN supports 2 through 256 ranks")
        self.device = torch.device(getattr(nccl_comm, "device", "cpu"))
        if device is not None:
            chosen = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
            if chosen.type != self.device.type or (chosen.index is not None and chosen != self.device):
                raise ValueError("Context and NCCL communicator must use the same CUDA device")
        owners = [owner for owner in (expert_to_rank.tolist() if isinstance(expert_to_rank, torch.Tensor)
                                      else expert_to_rank)]
        if (not owners or config.topk > len(owners) or
                any(isinstance(o, bool) or not isinstance(o, int) or not 0 <= o < self.world_size for o in owners)):
            raise ValueError("invalid expert placement or topk")
        if config.diagnostics:
            raise NotImplementedError("host-ring diagnostics do not describe the GIN transport")
        if self.world_size * config.max_tokens_per_rank >= 1 << 31:
            raise ValueError("aggregate token capacity must fit int32")
        self.expert_to_rank = tuple(owners)
        self._id = uuid.uuid4().hex
        self._lock = threading.RLock()
        self._counter = 0
        self._closed = False
        self._failed = None
        self._outstanding = set()
        self.effective_channels = config.channels

        identity = node_identity()
        signatures = nccl_comm.all_gather_object((identity, asdict(config), self.expert_to_rank))
        if any(other[1:] != signatures[self.rank][1:] for other in signatures):
            raise ValueError("ranks must use matching configuration and expert placement")
        self.local_ranks = tuple(r for r, other in enumerate(signatures) if other[0] == identity)
        nodes = len({other[0] for other in signatures})
        gpu_bytes = config.gin_registered_bytes(self.world_size)
        if gpu_bytes > config.gin_gpu_budget_bytes:
            raise ValueError(f"GIN staging requires {gpu_bytes} GPU bytes per rank; increase budgets or reduce "
                             "token capacity")
        self.transport_info = {"nodes": nodes, "local_ranks": list(self.local_ranks), "gpu_bytes": gpu_bytes,
                               "wire": "grouped point-to-point transfers on the borrowed communicator"}
        local_index, seen = [], [0] * self.world_size
        for owner in owners:
            local_index.append(seen[owner])
            seen[owner] += 1
        self._owner = torch.tensor(owners + [self.world_size], dtype=torch.int64, device=self.device)
        self._local_index = torch.tensor(local_index + [-1], dtype=torch.int64, device=self.device)
        self._comm.barrier()

    # ------------------------------------------------------------------ helpers
    def _check_usable(self):
        if self._closed:
            raise RuntimeError("Context is closed")
        if self._failed is not None:
            raise RuntimeError("EP context is in a failed state; restart the worker group") from self._failed

    def _fail(self, error):
        self._failed = error
        return error

    def _input(self, what, value, dtype, *shape):
        """A contiguous inference tensor of exactly this dtype and shape on the context device."""
        problem = None
        if not isinstance(value, torch.Tensor):
            problem = "is not a tensor"
        elif value.device != self.device:
            problem = f"lives on {value.device}, the context on {self.device}"
        elif value.dtype != dtype or value.shape != torch.Size(shape):
            problem = f"is {value.dtype} {tuple(value.shape)}, expected {dtype} {shape}"
        elif value.requires_grad:
            problem = "requires grad; only inference tensors are accepted"
        if problem:
            raise ValueError(f"{what} {problem}")
        return value if value.is_contiguous() else value.contiguous()

    def _exchange_counts(self, row: torch.Tensor) -> torch.Tensor:
        """Everybody's row of int64 values: the result is the [world, len(row)] matrix."""
        send = [row for _ in range(self.world_size)]
        recv = [torch.empty_like(row) for _ in range(self.world_size)]
        self._comm.exchange(send, recv)
        return torch.stack(recv)

    # ---------------------------------------------------------------- workspaces
    def create_workspace(self, recv_capacity, local_tokens, *, fused_combine=False):
        bounds = {"recv_capacity": (recv_capacity, self.world_size * self.config.max_tokens_per_rank),
                  "local_tokens": (local_tokens, self.config.max_tokens_per_rank)}
        for name, (value, limit) in bounds.items():
            if type(value) is not int or value < 0 or value > limit:
                raise ValueError(f"invalid workspace capacity: {name} must be an integer in [0, {limit}]")
        if self.device.type == "cuda" and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("workspaces are allocated outside CUDA Graph capture")
        return MultiNodeWorkspace(self, recv_capacity, local_tokens, fused_combine)

    # ------------------------------------------------------------------ dispatch
    def _dispatch(self, x, topk_ids, topk_weights, tag, recv_capacity, workspace, fused_combine, active_channels):
        cfg, world = self.config, self.world_size
        with self._lock:
            self._check_usable()
            if self.device.type == "cuda" and torch.cuda.is_current_stream_capturing():
                raise RuntimeError("the multi-node transport reads transfer sizes on the host and cannot be captured")
            if not isinstance(x, torch.Tensor) or x.ndim != 2:
                raise ValueError("hidden must be a BF16 [tokens, hidden] tensor")
            n = x.shape[0]
            if n > cfg.max_tokens_per_rank:
                raise ValueError("local token capacity exceeded")
            if len(self._outstanding) >= cfg.max_pending_operations:
                raise RuntimeError("combine earlier handles before submitting more dispatches")
            capacity = recv_capacity
            if capacity is None:
                capacity = workspace.recv_capacity if workspace is not None else world * cfg.max_tokens_per_rank
            if workspace is None:
                workspace = self.create_workspace(capacity, n, fused_combine=fused_combine)
            if (not isinstance(workspace, MultiNodeWorkspace) or workspace.context_id != self._id or
                    workspace.recv_capacity != capacity or workspace.local_tokens != n or workspace.busy):
                raise ValueError("workspace ownership, capacity or lifetime mismatch")
            hidden = self._input("hidden", x, torch.bfloat16, n, cfg.hidden_size)
            if not isinstance(topk_ids, torch.Tensor) or topk_ids.dtype not in (torch.int32, torch.int64):
                raise ValueError("topk_ids must be int32 or int64")
            ids = self._input("topk_ids", topk_ids, topk_ids.dtype, n, cfg.topk).to(torch.int64)
            weights = self._input("topk_weights", topk_weights, torch.float32, n, cfg.topk)

            # ---- route: destination columns, validation ------------------------------------
            experts = len(self.expert_to_rank)
            active = ids >= 0
            in_range = active & (ids < experts)
            bad = ((ids < -1) | (ids >= experts)).any() | (active & ~torch.isfinite(weights)).any()
            if cfg.topk > 1 and n:
                ordered, _ = torch.sort(torch.where(active, ids, -1 - torch.arange(cfg.topk, device=self.device)), dim=1)
                bad = bad | (ordered[:, 1:] == ordered[:, :-1]).any()           # an expert twice in one row
            safe = torch.where(in_range, ids, torch.full_like(ids, experts))    # column `experts` = nowhere
            owner = self._owner[safe]                                           # world = nowhere
            hit = torch.zeros((n, world + 1), dtype=torch.bool, device=self.device)
            if n:
                hit.scatter_(1, owner, True)
            hit = hit[:, :world]
            sent_tokens = [torch.nonzero(hit[:, r], as_tuple=False).flatten() for r in range(world)]
            row = torch.tensor([t.numel() for t in sent_tokens] + [0], dtype=torch.int64)
            row[-1] = int(bad)
            matrix = self._exchange_counts(row.to(self.device)).cpu()            # the one host read-back
            if bool(matrix[:, -1].any()):
                culprits = [r for r in range(world) if matrix[r, -1]]
                raise self._fail(RuntimeError(f"host_sm: {ERROR_TEXT[1]} (ranks {culprits})"))
            totals = matrix[:, :world].sum(dim=0)
            # Every rank knows every rank's capacity only if all use the same bound: the default
            # and scheduler-derived capacities are the same everywhere; a rank checks its own.
            overflow = torch.zeros(1, dtype=torch.int64)
            overflow[0] = int(totals[self.rank] > capacity)
            verdict = self._exchange_counts(overflow.to(self.device)).cpu()
            if bool(verdict.any()):
                culprits = [r for r in range(world) if verdict[r, 0]]
                raise self._fail(RuntimeError(f"host_sm: {ERROR_TEXT[2]} (ranks {culprits})"))
            received = [int(v) for v in matrix[:, self.rank]]

            # ---- records: row | local ids | weights | token, packed as bytes ----------------
            k, h = cfg.topk, cfg.hidden_size
            stride = h * 2 + k * 8 + k * 4 + 8
            send, recv = [], []
            for r in range(world):
                tokens = sent_tokens[r]
                mine = owner[tokens] == r
                local_ids = torch.where(mine, self._local_index[safe[tokens]], torch.full_like(ids[tokens], -1))
                local_weights = torch.where(mine, weights[tokens], torch.zeros_like(weights[tokens]))
                record = torch.cat([hidden[tokens].view(torch.uint8), local_ids.contiguous().view(torch.uint8),
                                    local_weights.contiguous().view(torch.uint8),
                                    tokens.to(torch.int64).unsqueeze(1).contiguous().view(torch.uint8)], dim=1)
                send.append(record.contiguous())
                recv.append(torch.empty((received[r], stride), dtype=torch.uint8, device=self.device))
            self._comm.exchange(send, recv)

            # ---- unpack in (source rank, token) order; reset the padding ----------------------
            total = sum(received)
            rows = torch.cat(recv) if total else torch.empty((0, stride), dtype=torch.uint8, device=self.device)
            at = 0
            workspace.hidden[:total] = rows[:, at:at + 2 * h].contiguous().view(torch.bfloat16)
            at += 2 * h
            workspace.local_ids[:total] = rows[:, at:at + 8 * k].contiguous().view(torch.int64)
            at += 8 * k
            workspace.weights[:total] = rows[:, at:at + 4 * k].contiguous().view(torch.float32)
            at += 4 * k
            source = torch.repeat_interleave(torch.arange(world, device=self.device),
                                             torch.tensor(received, device=self.device))
            workspace.inverse[:total, 0] = source
            workspace.inverse[:total, 1] = rows[:, at:at + 8].contiguous().view(torch.int64).flatten()
            workspace.hidden[total:] = 0
            workspace.local_ids[total:] = -1
            workspace.weights[total:] = 0
            workspace.inverse[total:] = -1
            workspace.count[0] = total

            self._counter += 1
            workspace.generation += 1
            workspace.busy = True
            route = _Route(workspace, workspace.generation, sent_tokens, received, workspace.inverse, workspace.count,
                           active_channels or self.effective_channels)
            handle = RouteHandle(self._id, self._counter, route, n, capacity, tag)
            self._outstanding.add(handle.operation)
            metrics = {"sent_rows": int(row[:world].sum()), "received_rows": total, "record_bytes": stride}
            return DispatchBatch(workspace.hidden, workspace.local_ids, workspace.weights, handle,
                                 workspace.count), metrics

    def dispatch_on_stream(self, x, topk_ids, topk_weights, tag=None, stream=None, recv_capacity=None,
                           active_channels=None, workspace=None, fused_combine=False):
        return self._on_stream(stream, self._dispatch, x, topk_ids, topk_weights, tag, recv_capacity, workspace,
                               fused_combine, active_channels)[0]

    def dispatch_async(self, x, topk_ids, topk_weights, tag=None, stream=None, recv_capacity=None,
                       active_channels=None, workspace=None, fused_combine=False):
        batch, metrics = self._on_stream(stream, self._dispatch, x, topk_ids, topk_weights, tag, recv_capacity,
                                         workspace, fused_combine, active_channels)
        return CompletedTicket(batch, metrics)

    def _on_stream(self, stream, operation, *arguments):
        if self.device.type != "cuda":
            return operation(*arguments)
        with torch.cuda.device(self.device), torch.cuda.stream(stream or torch.cuda.current_stream(self.device)):
            return operation(*arguments)

    # ------------------------------------------------------------------- combine
    def _combine(self, partial, handle, tag, weights_applied):
        cfg, world = self.config, self.world_size
        with self._lock:
            self._check_usable()
            if (not isinstance(handle, RouteHandle) or handle._context_id != self._id or handle._consumed or
                    handle.operation not in self._outstanding):
                raise ValueError("combine requires an unconsumed handle from this context")
            if weights_applied is not True:
                raise ValueError("expert partials must already contain routing weights")
            if tag != handle.tag:
                raise ValueError("combine tag differs from dispatch")
            route, n, capacity = handle._plan, handle.local_token_count, handle.received_count
            workspace = route.workspace
            if workspace.generation != route.generation:
                raise RuntimeError("dispatch workspace was reused before combine")
            total = sum(route.received)
            if (not isinstance(partial, torch.Tensor) or partial.device != self.device or
                    partial.dtype != torch.bfloat16 or partial.ndim != 2 or partial.shape[1] != cfg.hidden_size or
                    not total <= partial.shape[0] <= capacity or partial.requires_grad):
                raise ValueError("partial has invalid shape or dtype")
            partial = partial.contiguous()
            send, recv, at = [], [], 0
            for r in range(world):
                send.append(partial[at:at + route.received[r]].contiguous())
                at += route.received[r]
                recv.append(torch.empty((route.sent_tokens[r].numel(), cfg.hidden_size), dtype=torch.bfloat16,
                                        device=self.device))
            self._comm.exchange(send, recv)
            # Rank-order FP32 accumulation; each rank contributes at most one row per token, so
            # index_add_ adds exactly one value per element and the order is the loop's.
            accumulator = torch.zeros((n, cfg.hidden_size), dtype=torch.float32, device=self.device)
            single = cfg.single_rounding
            for r in range(world):
                if r == self.rank and not single:
                    continue
                accumulator.index_add_(0, route.sent_tokens[r], recv[r].float())
            if not single:
                accumulator = accumulator.to(torch.bfloat16).float()
                accumulator.index_add_(0, route.sent_tokens[self.rank], recv[self.rank].float())
            workspace.output[:n] = accumulator.to(torch.bfloat16)
            handle._consumed = True
            self._outstanding.remove(handle.operation)
            workspace.busy = False
            return workspace.output[:n], {"returned_rows": total}

    def combine_on_stream(self, partial, handle, tag=None, stream=None, weights_applied=True):
        return self._on_stream(stream, self._combine, partial, handle, tag, weights_applied)[0]

    def combine_async(self, partial, handle, tag=None, stream=None, weights_applied=True):
        return CompletedTicket(*self._on_stream(stream, self._combine, partial, handle, tag, weights_applied))

    # ----------------------------------------------------------------- lifecycle
    def enable_cuda_graph(self):
        raise NotImplementedError("the multi-node transport reads transfer sizes on the host; its operations "
                                  "cannot be captured into CUDA graphs")

    def check_errors(self):
        with self._lock:
            self._check_usable()
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)

    def close(self):
        with self._lock:
            if self._closed:
                return
            if self._failed is None:
                if self._outstanding:
                    raise RuntimeError("combine outstanding handles before closing")
                if self.device.type == "cuda":
                    torch.cuda.synchronize(self.device)
                self._comm.barrier()
            self._closed = True
