"""Validated resource limits of one expert-parallel group.

Field names, defaults and validation follow the reference's ``Config``
(ep_xpress/config.py:9-93) so that existing call sites keep working; what is
new is the ``"nvlink"`` transport (default) whose payloads never leave GPU
memory, and the sizing helpers of its peer-mapped HBM heap. The host-layout
helpers (``chunk_rows``, ``slot_bytes``, ``pool_bytes`` ...) describe the
host-staged ``host_ce`` transport kept as the CPU-visible oracle path.

``transport="host_sm"`` is accepted for source compatibility: its contract
(padded receive tensors, device ``valid_count``, borrowed workspaces, CUDA
graph replay) is exactly the contract of the NVLink transport, so it selects
the same device kernels; nothing is staged through host memory.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

DEVICE_TRANSPORTS = ("nvlink", "host_sm")
_TRANSPORTS = ("nvlink", "host_sm", "host_ce")
_CTRL_HEADER_BYTES = 256
_SLOT_ALIGN = 256
_ROUTE_TILE = 512
_FLAG_LINE = 128          # arrival words behind every staging row (csrc/epx_layout.h)


def _round_up(value: int, alignment: int) -> int:
    return (value + alignment - 1) // alignment * alignment


def _is_int(value) -> bool:
    return isinstance(value, int) and not isinstance(value, bool)


@dataclass(frozen=True)
class Config:
    hidden_size: int
    topk: int
    max_tokens_per_rank: int
    chunk_bytes: int = 2 << 20
    slots: int = 2
    host_pool_budget_bytes: int = 512 << 20
    timeout_seconds: float = 60.0
    poll_interval_seconds: float = 0.0001
    max_pending_operations: int = 8
    workload: str = "auto"
    transport: str = "nvlink"
    combine_backend: str = "gpu"
    graph_mode: str = "eager"
    fatal_errors: bool = False
    channels: int = 4
    diagnostics: bool = False
    combine_frame_rows: int = 0
    decode_max_tokens: int = 0
    combine_warp_specialization: bool = False
    decode_single_frame: bool = False
    internode_transport: str = "none"
    gin_contexts: int = 4
    gin_gpu_budget_bytes: int = 2 << 30
    # --- NVLink transport -------------------------------------------------
    gpu_pool_budget_bytes: int = 16 << 30     # bound of the peer-mapped heap of one rank
    workspace_pool_bytes: int = 0             # heap reserve for create_workspace; 0 = two more slots
    combine_rounding: str = "auto"            # "two_step" (single-node reference), "single" (multi-node reference); auto: by transport
    zero_padding: bool = True                 # keep activation rows above valid_count at zero
    cooperative_launch: bool = True           # driver-guaranteed co-residency of the transport CTAs
    debug_delay_ns: int = 0                   # debugging: random sleeps below this bound at kernel phase boundaries
    combine_streaming: str = "auto"           # "auto"/"on": mailbox protocol (reduce while peers still push); "off": push, signal, reduce

    @property
    def single_rounding(self) -> bool:
        """One rounding over all ranks (the multi-node formula) instead of remote-sum, round, add local, round."""
        if self.combine_rounding == "auto":
            return self.internode_transport == "gin"
        return self.combine_rounding == "single"

    @property
    def device_transport(self) -> bool:
        return self.transport in DEVICE_TRANSPORTS

    def inert_fields(self) -> tuple:
        """Fields that were given a non-default value but change nothing on the chosen transport.

        The reference's host-staged device transport needs these knobs (frame sizes, warp
        specialisation of its pair combine, single-frame dispatch, a trap on errors, the host
        loop's poll interval); the NVLink transport has no frames to size and selects its kernel
        variants by shape. They stay accepted so that existing call sites keep working; a context
        warns once when it is constructed with any of them set.
        """
        if not self.device_transport:
            return ()
        defaults = {"chunk_bytes": 2 << 20, "combine_frame_rows": 0, "combine_warp_specialization": False,
                    "decode_single_frame": False, "workload": "auto", "poll_interval_seconds": 0.0001,
                    "host_pool_budget_bytes": 512 << 20}
        return tuple(name for name, default in defaults.items() if getattr(self, name) != default)

    def __post_init__(self):
        device = self.transport in DEVICE_TRANSPORTS
        if self.internode_transport not in ("none", "gin"):
            raise ValueError("internode_transport must be none or gin")
        if self.internode_transport == "gin" and self.transport != "host_sm":
            raise ValueError("GIN requires host_sm for intra-node payloads")
        if not _is_int(self.gin_contexts) or not 1 <= self.gin_contexts <= 32:
            raise ValueError("gin_contexts must be an integer in [1, 32]")
        if not _is_int(self.gin_gpu_budget_bytes) or self.gin_gpu_budget_bytes <= 0:
            raise ValueError("gin_gpu_budget_bytes must be positive")
        for name in ("decode_single_frame", "combine_warp_specialization", "fatal_errors", "diagnostics",
                     "zero_padding", "cooperative_launch"):
            if not isinstance(getattr(self, name), bool):
                raise ValueError(f"{name} must be a bool")
        if self.decode_single_frame and (not device or not self.decode_max_tokens):
            raise ValueError("decode_single_frame requires host_sm with decode_max_tokens")
        for name in ("combine_warp_specialization", "fatal_errors", "diagnostics"):
            if getattr(self, name) and not device:
                raise ValueError(f"{name} is only supported by host_sm")
        for name in ("hidden_size", "topk", "max_tokens_per_rank", "chunk_bytes", "slots",
                     "host_pool_budget_bytes", "max_pending_operations", "channels", "gpu_pool_budget_bytes"):
            value = getattr(self, name)
            if not _is_int(value) or value <= 0:
                raise ValueError(f"{name} must be a positive integer")
        if not _is_int(self.workspace_pool_bytes) or self.workspace_pool_bytes < 0:
            raise ValueError("workspace_pool_bytes must be a nonnegative integer")
        if self.channels > 32:
            raise ValueError("channels must be at most 32")
        for name, maximum in (("combine_frame_rows", 256), ("decode_max_tokens", 256)):
            value = getattr(self, name)
            if not _is_int(value) or not 0 <= value <= maximum:
                raise ValueError(f"{name} must be an integer in [0, {maximum}]")
            if value and not device:
                raise ValueError(f"{name} is only supported by host_sm")
        if self.chunk_bytes < self.hidden_size * 2:
            raise ValueError("chunk_bytes must fit at least one BF16 row")
        if not isinstance(self.timeout_seconds, (int, float)) or isinstance(self.timeout_seconds, bool) \
                or not math.isfinite(self.timeout_seconds) or self.timeout_seconds <= 0:
            raise ValueError("timeout_seconds must be finite and positive")
        if not isinstance(self.poll_interval_seconds, (int, float)) or isinstance(self.poll_interval_seconds, bool) \
                or not math.isfinite(self.poll_interval_seconds) or self.poll_interval_seconds < 0:
            raise ValueError("poll_interval_seconds must be finite and nonnegative")
        if self.workload not in ("auto", "prefill", "decode"):
            raise ValueError("workload must be auto, prefill, or decode")
        if self.transport not in _TRANSPORTS:
            raise NotImplementedError("transport must be nvlink, host_sm or host_ce")
        if self.combine_rounding not in ("auto", "two_step", "single"):
            raise ValueError("combine_rounding must be auto, two_step or single")
        if not _is_int(self.debug_delay_ns) or not 0 <= self.debug_delay_ns <= 1_000_000:
            raise ValueError("debug_delay_ns must be an integer in [0, 1000000]")
        if self.combine_streaming not in ("auto", "on", "off"):
            raise ValueError("combine_streaming must be auto, on or off")
        if device:
            # Limits of the device kernels: rows are moved as BF16 pairs, row indices and byte
            # offsets are 32-bit in places, waits are timed in 64-bit nanoseconds.
            int32_max = (1 << 31) - 1
            limits = (("topk <= 256", self.topk <= 256), ("slots <= 64", self.slots <= 64),
                      ("chunk_rows <= 65536", self.chunk_rows <= 65536),
                      ("an even hidden size below 2^31", self.hidden_size % 2 == 0 and self.hidden_size <= int32_max),
                      ("timeout_seconds <= 3600", self.timeout_seconds <= 3600),
                      ("max_tokens_per_rank below 2^31", self.max_tokens_per_rank <= int32_max))
            broken = [rule for rule, holds in limits if not holds]
            if broken:
                raise ValueError("the device transports need " + ", ".join(broken))
        if self.combine_backend != "gpu":
            raise NotImplementedError("this release implements GPU combine only")
        if self.graph_mode != "eager":
            raise NotImplementedError("CUDA Graph capture is enabled through enable_cuda_graph(), not graph_mode")

    # ---- host-staged (host_ce) wire layout ---------------------------------
    @property
    def chunk_rows(self) -> int:
        return self.chunk_bytes // (self.hidden_size * 2)

    @property
    def slot_bytes(self) -> int:
        return _round_up(self.chunk_rows * self.hidden_size * 2, 4096)

    def channel_chunk_rows(self, channels=None) -> int:
        channels = self.channels if channels is None else channels
        return max(1, -(-self.chunk_rows // channels))

    def combine_chunk_rows(self, channels=None, queue_peers=1) -> int:
        if not _is_int(queue_peers) or not 1 <= queue_peers <= 63:
            raise ValueError("queue_peers must be an integer in [1, 63]")
        if self.combine_frame_rows:
            return self.combine_frame_rows
        return max(1, -(-self.channel_chunk_rows(channels) // queue_peers))

    def pool_bytes(self, world_size, *, local_world_size=None) -> int:
        """Host memory of the host-staged transport: one send ring per rank and phase."""
        if self.internode_transport == "gin":
            if not _is_int(local_world_size) or not _is_int(world_size) or local_world_size >= world_size:
                raise ValueError("GIN host budgeting requires this node's local_world_size < world_size")
            return local_world_size * self.gin_producer_bytes(local_world_size)
        _check_world(world_size)
        if self.device_transport:
            return 0
        return 2 * world_size * self.slots * (self.slot_bytes + 4096)

    def pinned_working_set_bytes(self, world_size, *, local_world_size=None) -> int:
        _check_world(world_size)
        if self.device_transport:
            return 0
        packs = world_size * (world_size - 1) * self.slots * self.chunk_rows * self.hidden_size * 2
        return self.pool_bytes(world_size) + packs

    # ---- NVLink heap layout (mirrors csrc/epx_layout.h) ---------------------
    def ctrl_bytes(self, world_size) -> int:
        _check_world(world_size)
        w = world_size
        words = 2 * w * w + 2 * w * 8 + 2 * w + w + 2 * w
        hand = _round_up(_CTRL_HEADER_BYTES + words * 8 + w * 4, 256)       # hand-over slots of the push CTAs
        return _round_up(hand + 64 * (64 + 8 * 4 * 16), 4096)

    def nvlink_slot_bytes(self, world_size, capacity=None, tokens=None) -> int:
        """Bytes of one operation slot: receive planes, partial plane and route state."""
        _check_world(world_size)
        capacity = world_size * self.max_tokens_per_rank if capacity is None else capacity
        tokens = self.max_tokens_per_rank if tokens is None else tokens
        h, k, w = self.hidden_size, self.topk, world_size
        fanout = min(k, w)
        tiles = -(-tokens // _ROUTE_TILE)
        parts = (capacity * h * 2, capacity * k * 8, capacity * k * 4, capacity * 16, capacity * 4,
                 tokens * fanout * (h * 2 + _FLAG_LINE), capacity * h * 2,
                 tokens * 8, tokens * fanout * 4, tokens * fanout * 4, (tiles + 1) * w * 4, w * 8, w * 4, w * 4, w * 4, 64 * 4,
                 tokens * h * 2)
        return _round_up(sum(_round_up(p, _SLOT_ALIGN) for p in parts), 4096)

    def nvlink_slot_breakdown(self, world_size, capacity=None, tokens=None) -> dict:
        """Bytes of every plane of one operation slot, by name (the same arithmetic as
        :meth:`nvlink_slot_bytes`). ``hidden``/``ids``/``weights``/``inverse``/``ret`` are what peers
        store a dispatch into (``capacity`` rows), ``staging`` is where expert ranks push the rows
        of this rank's ``tokens`` (one row and one arrival line per (token, destination)),
        ``partial`` is the default output plane of the expert runner, ``output`` the combine
        result of a workspace, ``route_state`` the rank-local bookkeeping."""
        _check_world(world_size)
        capacity = world_size * self.max_tokens_per_rank if capacity is None else capacity
        tokens = self.max_tokens_per_rank if tokens is None else tokens
        h, k, w = self.hidden_size, self.topk, world_size
        fanout = min(k, w)
        tiles = -(-tokens // _ROUTE_TILE)
        up = lambda value: _round_up(value, _SLOT_ALIGN)      # noqa: E731
        parts = {"hidden": up(capacity * h * 2), "ids": up(capacity * k * 8), "weights": up(capacity * k * 4),
                 "inverse": up(capacity * 16), "ret": up(capacity * 4),
                 "staging": up(tokens * fanout * (h * 2 + _FLAG_LINE)), "partial": up(capacity * h * 2),
                 "route_state": (up(tokens * 8) + 2 * up(tokens * fanout * 4) + up((tiles + 1) * w * 4) + up(w * 8)
                                 + 3 * up(w * 4) + up(64 * 4)),
                 "output": up(tokens * h * 2)}
        parts["total"] = _round_up(sum(parts.values()), 4096)
        return parts

    def heap_bytes(self, world_size) -> int:
        """Peer-mapped HBM one rank allocates at bootstrap."""
        slot = self.nvlink_slot_bytes(world_size)
        reserve = self.workspace_pool_bytes or 2 * slot
        guards = 8192 * (self.slots + 16) if self.diagnostics else 0     # guard bands around every slot
        return _round_up(self.ctrl_bytes(world_size) + self.slots * slot + reserve + guards, 2 << 20)

    def mapped_arena_bytes(self, topk, channels=None, queue_peers=1, *, dispatch_banks=0) -> int:
        """Host-mapped queue bytes of one producer: always 0 here.

        The reference sizes a mapped ``/dev/shm`` arena per producer with this helper
        (ep_xpress/config.py:167-191). The device transports of this library stage nothing in
        host memory (``heap_bytes`` is their footprint, in HBM), so the answer is zero for every
        legal argument; the arguments are still validated so that budgeting code ported from
        the reference fails on the same mistakes.
        """
        if not _is_int(dispatch_banks) or dispatch_banks not in (0, 2):
            raise ValueError("dispatch_banks must be 0 or 2")
        if dispatch_banks and not topk:
            raise ValueError("extra dispatch banks are only valid for dispatch")
        if not _is_int(queue_peers) or not 1 <= queue_peers <= 63 or (topk and queue_peers != 1):
            raise ValueError("queue_peers must be in [1, 63] and dispatch requires one queue")
        return 0

    # ---- multi-node (GIN) staging layout: sizing only, the transport itself is gated ----------
    def _gin_record_bytes(self) -> int:
        """One dispatch record on the wire: BF16 row, K int32 ids, K fp32 weights, token index."""
        return _round_up(self.hidden_size * 2 + self.topk * 8 + 4, 128)

    def gin_producer_bytes(self, local_world_size) -> int:
        """Host bytes one producer needs on its node: its dispatch records (read by the node's
        other ranks) followed by one combine row slot per (local peer, token).
        Same arithmetic as ep_xpress/config.py:103-112."""
        if not _is_int(local_world_size) or not 1 <= local_world_size <= 256:
            raise ValueError("local_world_size must be an integer in [1, 256]")
        records = _round_up(128 + self.max_tokens_per_rank * self._gin_record_bytes(), 4096)
        rows = local_world_size * self.max_tokens_per_rank * self.hidden_size * 2
        return _round_up(records + rows, 4096)

    def gin_registered_bytes(self, world_size) -> int:
        """GPU bytes one rank registers with the network: a count header, a send window plus one
        receive window per rank of dispatch records, and FP32-wide combine rows per source rank,
        rounded to 2 MiB registration granules (ep_xpress/config.py:114-123)."""
        if not _is_int(world_size) or not 2 <= world_size <= 256:
            raise ValueError("GIN world_size must be an integer in [2, 256]")
        header = _round_up(world_size * 8, 128)
        windows = (world_size + 1) * self.max_tokens_per_rank * self._gin_record_bytes()
        rows = world_size * self.max_tokens_per_rank * self.hidden_size * 4
        return _round_up(header + windows + rows, 2 << 20)

    def mailbox_arena_bytes(self, world_size, *, packet_rows=0) -> int:
        """Decode mailboxes are ordinary slots of the heap; no separate arena exists."""
        _check_world(world_size)
        if not self.decode_max_tokens:
            return 0
        return self.nvlink_slot_bytes(world_size, world_size * self.decode_max_tokens, self.decode_max_tokens)


def _check_world(world_size):
    if not _is_int(world_size) or not 1 <= world_size <= 63:
        raise ValueError("world_size must be an integer in [1, 63]")
