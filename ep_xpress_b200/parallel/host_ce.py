"""The host-staged ``host_ce`` transport: the CPU-visible oracle path.

Payloads travel through bounded shared-memory rings (``csrc/host_ring.cpp``) in
chunks of ``Config.chunk_rows`` rows; every operation first exchanges its router
output over the control plane and plans routes on the CPU
(:func:`ep_xpress_b200.utils.routing.plan_routes`). It is slow by construction and
exists for the reasons the reference keeps its own ``host_ce``
(ep_xpress/context.py:122-444, ep_xpress/transport.py:15-186): an exact,
inspectable statement of the semantics, usable without NVLink - and here even
without a GPU, because it accepts CPU tensors and any ``ControlPlane`` (e.g. a
gloo group).

Contract differences from the device transports (same as the reference): outputs
are exact-size, ``valid_count`` is a Python int, rows are ordered by (source
rank, token), ``recv_capacity``/``workspace`` are rejected, operations run
synchronously on the calling thread and the returned ticket is already complete.
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
import tempfile
import threading
import time
import uuid
from dataclasses import asdict

import torch

from ..comm import ControlPlane
from ..context import Context, DispatchBatch, RouteHandle
from ..utils import routing


class CompletedTicket:
    """Ticket of a synchronous operation; ``wait`` only hands the value over."""

    def __init__(self, value, metrics):
        self._value, self._metrics = value, metrics

    def wait(self, stream=None, timeout=None):
        return self._value

    @property
    def done(self):
        return True

    @property
    def metrics(self):
        return dict(self._metrics)


def _tag_digest(tag):
    return hashlib.sha256(json.dumps(tag, sort_keys=True, default=str).encode()).hexdigest()


class HostCEContext(Context):
    def __init__(self, nccl_comm, expert_to_rank, config, device=None, shared_directory=None):
        if not isinstance(nccl_comm, ControlPlane):
            raise TypeError("nccl_comm must be an NCCLCommHandle or another ControlPlane")
        from .. import native as native_loader
        self._native = native_loader.load()
        self.config, self._comm = config, nccl_comm
        self.rank, self.world_size = nccl_comm.rank, nccl_comm.world_size
        if not 1 <= self.world_size <= 63:
            raise ValueError("the EP group must have between 1 and 63 ranks")
        self.expert_to_rank = [int(owner) for owner in expert_to_rank]
        if not self.expert_to_rank or any(not 0 <= o < self.world_size for o in self.expert_to_rank):
            raise ValueError("expert_to_rank must map every expert to a rank of the group")
        if config.topk > len(self.expert_to_rank):
            raise ValueError("topk exceeds the number of experts")
        self.device = torch.device(device) if device is not None else torch.device(getattr(nccl_comm, "device", "cpu"))
        self._id = uuid.uuid4().hex
        self._lock = threading.RLock()
        self._counter = 0
        self._failed = None
        self._closed = False
        signature = {"config": asdict(config), "placement": tuple(self.expert_to_rank), "world": self.world_size}
        if any(other != signature for other in nccl_comm.all_gather_object(signature)):
            raise ValueError("EP ranks were constructed with a different configuration or placement")
        budget = config.pool_bytes(self.world_size)
        if budget > config.host_pool_budget_bytes:
            raise ValueError("negotiated host rings exceed host_pool_budget_bytes")
        root = None
        if self.rank == 0:
            parent = shared_directory or ("/dev/shm" if os.path.isdir("/dev/shm") else tempfile.gettempdir())
            root = tempfile.mkdtemp(prefix="epx_b200_", dir=parent)
        self._root = nccl_comm.all_gather_object(root)[0]
        self._rings = {"dispatch": [None] * self.world_size, "combine": [None] * self.world_size}
        error = None
        try:
            for phase in self._rings:
                self._rings[phase][self.rank] = self._native.HostRing(self._path(phase, self.rank), config.slots,
                                                                      config.slot_bytes, True)
        except Exception as exc:
            error = repr(exc)
        errors = [e for e in nccl_comm.all_gather_object(error) if e]
        if errors:
            self._release()
            raise RuntimeError("host ring allocation failed: " + "; ".join(errors))
        for phase in self._rings:
            for peer in range(self.world_size):
                if peer != self.rank:
                    self._rings[phase][peer] = self._native.HostRing(self._path(phase, peer))
        nccl_comm.barrier()

    def _path(self, phase, rank):
        return os.path.join(self._root, f"{phase}_{rank}.ring")

    # ---------------------------------------------------------------- health
    def _check_usable(self):
        if self._closed:
            raise RuntimeError("EP context is closed")
        if self._failed is not None:
            raise RuntimeError("EP context is in a failed state") from self._failed

    def _abort(self, error):
        if self._failed is None:
            self._failed = error
            for ring in (self._rings["dispatch"][self.rank], self._rings["combine"][self.rank]):
                if ring is not None:
                    ring.abort()

    def check_errors(self):
        self._check_usable()
        for phase in self._rings:
            for ring in self._rings[phase]:
                if ring is not None and ring.aborted():
                    error = RuntimeError("host_ce: a peer aborted the operation")
                    self._abort(error)
                    raise error

    def _metadata(self, phase, tag, payload, error=None):
        """Cross-check (operation, phase, tag) on every rank and exchange per-op metadata."""
        self._counter += 1
        mine = {"operation": self._counter, "phase": phase, "tag": _tag_digest(tag), "error": error,
                "payload": payload}
        gathered = self._comm.all_gather_object(mine)
        failures = [f"rank {r}: {g['error']}" for r, g in enumerate(gathered) if g["error"]]
        if failures:
            raise ValueError("; ".join(failures))
        if any((g["operation"], g["phase"], g["tag"]) != (mine["operation"], phase, mine["tag"]) for g in gathered):
            raise RuntimeError("host_ce: operation identity (tag or order) mismatch between ranks")
        return [g["payload"] for g in gathered]

    # ---------------------------------------------------------------- exchange
    def _exchange(self, phase, operation, rows_cpu, send_masks, recv_plan):
        """Simultaneous send/receive of row chunks.

        ``send_masks[c]``: bitmask of ranks that read chunk ``c`` of my rows (0 = not sent).
        ``recv_plan[s]``: list of (chunk, row indices inside the chunk) I need from rank ``s``.
        Returns {source: [rows tensor per needed chunk]} and metrics.
        """
        cfg = self.config
        chunk_rows, row_bytes = cfg.chunk_rows, rows_cpu.shape[1] * rows_cpu.element_size() if rows_cpu.numel() else 0
        mine = self._rings[phase][self.rank]
        send_queue = [c for c, mask in enumerate(send_masks) if mask]
        received = {s: [] for s in recv_plan}
        cursors = {s: 0 for s in recv_plan}
        raw = rows_cpu.contiguous().view(torch.uint8).reshape(rows_cpu.shape[0], -1) if rows_cpu.numel() else None
        metrics = {"chunks_sent": 0, "chunks_received": 0, "bytes_sent": 0, "bytes_received": 0,
                   "poll_iterations": 0, "backpressure_iterations": 0}
        deadline = time.monotonic() + cfg.timeout_seconds
        while send_queue or any(cursors[s] < len(recv_plan[s]) for s in recv_plan):
            progressed = False
            if send_queue:
                chunk = send_queue[0]
                slot = mine.try_claim((operation << 32) | chunk, send_masks[chunk])
                if slot >= 0:
                    part = raw[chunk * chunk_rows:(chunk + 1) * chunk_rows]
                    mine.payload(slot)[:part.numel()].copy_(part.reshape(-1))
                    mine.publish(slot, part.shape[0])
                    send_queue.pop(0)
                    metrics["chunks_sent"] += 1
                    metrics["bytes_sent"] += part.numel()
                    progressed = True
                else:
                    metrics["backpressure_iterations"] += 1
            # Incoming data is always drained, also while my own slots are full.
            for source, needs in recv_plan.items():
                if cursors[source] >= len(needs):
                    continue
                chunk, picks = needs[cursors[source]]
                ring = self._rings[phase][source]
                generation = (operation << 32) | chunk
                for slot in range(ring.slots()):
                    rows = ring.ready(slot, generation)
                    if rows < 0:
                        continue
                    width = row_bytes_of(self.config, phase)
                    payload = ring.payload(slot)[:rows * width].reshape(rows, width)
                    received[source].append(payload[picks].clone())
                    ring.ack(slot, generation, self.rank)
                    cursors[source] += 1
                    metrics["chunks_received"] += 1
                    metrics["bytes_received"] += len(picks) * width
                    progressed = True
                    break
            metrics["poll_iterations"] += 1
            if not progressed:
                if time.monotonic() > deadline:
                    raise TimeoutError(f"host_ce {phase} timed out after {cfg.timeout_seconds} s")
                if cfg.poll_interval_seconds:
                    time.sleep(cfg.poll_interval_seconds)
        return received, metrics

    # ---------------------------------------------------------------- dispatch
    def dispatch_async(self, x, topk_ids, topk_weights, tag=None, stream=None, recv_capacity=None,
                       active_channels=None, workspace=None, fused_combine=False):
        if recv_capacity is not None or workspace is not None or active_channels is not None or fused_combine:
            raise ValueError("recv_capacity, workspace, active_channels and fused_combine are only supported by host_sm")
        with self._lock:
            self._check_usable()
            try:
                return self._dispatch(x, topk_ids, topk_weights, tag)
            except BaseException as error:
                self._abort(error)
                raise

    def _dispatch(self, x, topk_ids, topk_weights, tag):
        cfg = self.config
        if x.ndim != 2 or x.shape[1] != cfg.hidden_size or x.shape[0] > cfg.max_tokens_per_rank or \
                x.dtype != torch.bfloat16:
            raise ValueError("x must be BF16 [tokens, hidden] within the configured token capacity")
        ids_cpu = topk_ids.detach().cpu().to(torch.int64).reshape(-1, cfg.topk)
        weights_cpu = topk_weights.detach().cpu().to(torch.float32).reshape(-1, cfg.topk)
        error = None
        try:
            routing.plan_routes([ids_cpu], [weights_cpu], [0] * len(self.expert_to_rank), 1, cfg.topk)
        except ValueError as exc:
            error = str(exc)
        gathered = self._metadata("dispatch", tag, (ids_cpu, weights_cpu), error)
        plan = routing.plan_routes([g[0] for g in gathered], [g[1] for g in gathered], self.expert_to_rank,
                                   self.world_size, cfg.topk)
        operation = self._counter
        chunk_rows = cfg.chunk_rows
        x_cpu = x.detach().cpu()
        remote = plan.remote_masks()

        send_masks = [_or_all(remote[self.rank][c:c + chunk_rows])
                      for c in range(0, plan.token_counts[self.rank], chunk_rows)]
        recv_plan = {}
        for source in range(self.world_size):
            if source == self.rank:
                continue
            tokens = (plan.dest_rows[source][:, self.rank] >= 0).nonzero().flatten().tolist()
            needs = {}
            for t in tokens:
                needs.setdefault(t // chunk_rows, []).append(t % chunk_rows)
            if needs:
                recv_plan[source] = sorted(needs.items())
        received, metrics = self._exchange("dispatch", operation, x_cpu, send_masks, recv_plan)
        routes = plan.received[self.rank]
        parts = []
        for source in range(self.world_size):
            if source == self.rank:
                parts.append(x_cpu[routes.source_token[routes.source_rank == source]])
            elif source in received:
                rows = torch.cat(received[source]) if received[source] else torch.zeros((0, cfg.hidden_size * 2), dtype=torch.uint8)
                parts.append(rows.contiguous().view(torch.bfloat16).reshape(-1, cfg.hidden_size))
        hidden = torch.cat(parts) if parts else torch.zeros((0, cfg.hidden_size), dtype=torch.bfloat16)
        handle = RouteHandle(self._id, operation, plan, x.shape[0], routes.rows, tag)
        batch = DispatchBatch(hidden.to(self.device), routes.local_ids.to(self.device), routes.weights.to(self.device),
                              handle, routes.rows)
        return CompletedTicket(batch, metrics)

    # ---------------------------------------------------------------- combine
    def combine_async(self, partial, handle, tag=None, stream=None, weights_applied=True):
        with self._lock:
            self._check_usable()
            if weights_applied is not True:
                raise ValueError("combine accepts already-weighted rank partials only")
            if not isinstance(handle, RouteHandle) or handle._context_id != self._id:
                raise ValueError("handle belongs to another context")
            if handle._consumed:
                raise ValueError("handle has already been consumed by combine")
            try:
                value = self._combine(partial, handle, tag)
            except BaseException as error:
                self._abort(error)
                raise
            handle._consumed = True
            return value

    def _combine(self, partial, handle, tag):
        cfg, plan = self.config, handle._plan
        if partial.shape != (handle.received_count, cfg.hidden_size) or partial.dtype != torch.bfloat16:
            raise ValueError("partial must be BF16 [received rows, hidden]")
        self._metadata("combine", tag, handle.operation)
        operation = self._counter
        chunk_rows = cfg.chunk_rows
        partial_cpu = partial.detach().cpu()
        routes = plan.received[self.rank]
        owners = routes.source_rank
        send_masks = []
        for c in range(0, routes.rows, chunk_rows):
            mask = 0
            for owner in owners[c:c + chunk_rows].unique().tolist():
                if owner != self.rank:
                    mask |= 1 << owner
            send_masks.append(mask)
        recv_plan, token_order = {}, {}
        for dest in range(self.world_size):
            if dest == self.rank:
                continue
            rows = plan.dest_rows[self.rank][:, dest]
            tokens = (rows >= 0).nonzero().flatten()
            if not tokens.numel():
                continue
            needs = {}
            for t in tokens.tolist():
                r = int(rows[t])
                needs.setdefault(r // chunk_rows, []).append(r % chunk_rows)
            recv_plan[dest] = sorted(needs.items())
            token_order[dest] = tokens[torch.argsort(rows[tokens])]
        received, metrics = self._exchange("combine", operation, partial_cpu, send_masks, recv_plan)
        tokens_here = plan.token_counts[self.rank]
        single = cfg.single_rounding
        if partial.is_cuda:
            return CompletedTicket(self._reduce_on_gpu(partial, plan, received, token_order, tokens_here, single),
                                   metrics)
        remote = torch.zeros((tokens_here, cfg.hidden_size), dtype=torch.float32)
        local = torch.zeros((tokens_here, cfg.hidden_size), dtype=torch.float32)
        for dest in range(self.world_size):                    # ascending rank order
            if dest == self.rank:
                rows = plan.dest_rows[self.rank][:, dest]
                sel = (rows >= 0).nonzero().flatten()
                values = partial_cpu[rows[sel]].to(torch.float32)
                if single:
                    remote[sel] = remote[sel] + values
                else:
                    local[sel] = values
            elif dest in received:
                got = torch.cat(received[dest]).contiguous().view(torch.bfloat16).reshape(-1, cfg.hidden_size)
                sel = token_order[dest]
                remote[sel] = remote[sel] + got.to(torch.float32)
        if single:
            out = remote.to(torch.bfloat16)
        else:
            out = (remote.to(torch.bfloat16).to(torch.float32) + local).to(torch.bfloat16)
        return CompletedTicket(out.to(self.device), metrics)

    def _reduce_on_gpu(self, partial, plan, received, token_order, tokens_here, single):
        """Combine arithmetic on the GPU with the native helper kernels (the reference's host_ce
        does the same with its add_partial / finish_combine kernels, ep_xpress/context.py:375-408):
        every peer's rows are uploaded and accumulated into an FP32 plane in ascending rank
        order, then rounded, joined with the local rows and rounded again."""
        native, cfg, device = self._native, self.config, partial.device
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream(device).cuda_stream
            remote = torch.zeros((tokens_here, cfg.hidden_size), dtype=torch.float32, device=device)
            local = torch.zeros((tokens_here, cfg.hidden_size), dtype=torch.float32, device=device)
            status = torch.zeros(1, dtype=torch.int32, device=device)
            out = torch.empty((tokens_here, cfg.hidden_size), dtype=torch.bfloat16, device=device)
            for dest in range(self.world_size):                # ascending rank order
                if dest == self.rank:
                    rows = plan.dest_rows[self.rank][:, dest]
                    sel = (rows >= 0).nonzero().flatten()
                    if not sel.numel():
                        continue
                    values = partial.detach()[rows[sel].to(device)].contiguous()
                    native.add_partial(remote if single else local, values, sel.to(device), status, stream)
                elif dest in received:
                    got = torch.cat(received[dest]).contiguous().view(torch.bfloat16).reshape(-1, cfg.hidden_size)
                    native.add_partial(remote, got.to(device), token_order[dest].to(device), status, stream)
            native.finish_combine(remote, local, out, single, stream)
            if int(status.item()):
                raise RuntimeError("host_ce: a combine row index lies outside this rank's tokens")
        return out

    # ---------------------------------------------------------------- teardown
    def _release(self):
        for phase in self._rings:
            for rank, ring in enumerate(self._rings[phase]):
                if ring is not None:
                    ring.close()
            self._rings[phase] = [None] * self.world_size

    def close(self):
        with self._lock:
            if self._closed:
                return
            self._closed = True
            if self._failed is None:
                self._comm.barrier()
            self._release()
            if self.rank == 0 and self._root and os.path.isdir(self._root):
                shutil.rmtree(self._root, ignore_errors=True)


def _or_all(values):
    out = 0
    for v in values.tolist():
        out |= int(v)
    return out


def row_bytes_of(config, phase):
    return config.hidden_size * 2
