"""Borrowed NCCL communicator: the control plane of an EP context.

The library never creates a process group, never switches backend and never
destroys or aborts the communicator it is given (contract of the reference,
ep_xpress/comm.py:51-57 and tests/test_nccl_comm_cuda.py:46-73). The borrowed
``ncclComm_t`` is used for a handful of small all-gathers at context
construction and teardown: configuration signatures, CUDA IPC handles of the
peer-mapped heaps, launch-width negotiation. Token payloads never touch NCCL.

``ControlPlane`` is the minimal interface a context needs; ``NCCLCommHandle``
implements it over raw ``ncclAllGather`` calls on the owner's own NCCL DSO, and
``GroupControlPlane`` over any ``torch.distributed`` group (used by the
host-staged transport's CPU tests, where no NCCL exists).
"""

from __future__ import annotations

import ctypes
import pickle
import struct
import weakref
from pathlib import Path

import torch
import torch.distributed as dist

_MAX_METADATA_BYTES = 16 << 20
_NCCL_UINT8 = 1   # ncclUint8 in nccl.h's ncclDataType_t


class ControlPlane:
    """Rank, size and two collectives; everything a context bootstrap needs."""
    rank: int
    world_size: int

    def all_gather_object(self, value):
        raise NotImplementedError

    def barrier(self):
        self.all_gather_object(None)

    def exchange(self, send, recv):
        """Variable-size all-to-all on the current stream: ``send[r]`` goes to rank r,
        ``recv[r]`` is filled by rank r. Contiguous tensors of any dtype; the sizes must match
        pairwise, which the caller arranges with a fixed-size exchange of counts first. Only the
        multi-node transport moves payload this way."""
        raise NotImplementedError


class GroupControlPlane(ControlPlane):
    """Control plane over an existing torch.distributed group of any backend."""

    def __init__(self, group=None):
        if not dist.is_initialized():
            raise RuntimeError("initialize the process group first")
        self.group = dist.group.WORLD if group is None else group
        self.rank = dist.get_rank(self.group)
        self.world_size = dist.get_world_size(self.group)
        self.device = torch.device("cpu")

    def all_gather_object(self, value):
        gathered = [None] * self.world_size
        dist.all_gather_object(gathered, value, group=self.group)
        return gathered

    def exchange(self, send, recv):
        recv[self.rank].copy_(send[self.rank])
        ranks = dist.get_process_group_ranks(self.group)
        operations = []
        for peer in range(self.world_size):
            if peer == self.rank:
                continue
            if send[peer].numel():
                operations.append(dist.P2POp(dist.isend, send[peer], ranks[peer], group=self.group))
            if recv[peer].numel():
                operations.append(dist.P2POp(dist.irecv, recv[peer], ranks[peer], group=self.group))
        if operations:
            for work in dist.batch_isend_irecv(operations):
                work.wait()


class _NcclApi:
    """The NCCL entry points used, resolved from the owner's library only: three queries and
    ncclAllGather for the bootstrap, grouped ncclSend/ncclRecv for the multi-node transport."""

    def __init__(self, library_path):
        self._dso = ctypes.CDLL(str(library_path))
        void_p, c_int = ctypes.c_void_p, ctypes.c_int
        self._query = {}
        for name in ("ncclCommUserRank", "ncclCommCount", "ncclCommCuDevice"):
            fn = getattr(self._dso, name)
            fn.argtypes, fn.restype = [void_p, ctypes.POINTER(c_int)], c_int
            self._query[name] = fn
        self._all_gather = self._dso.ncclAllGather
        self._all_gather.argtypes = [void_p, void_p, ctypes.c_size_t, c_int, void_p, void_p]
        self._all_gather.restype = c_int
        self._error_string = self._dso.ncclGetErrorString
        self._error_string.argtypes, self._error_string.restype = [c_int], ctypes.c_char_p

    def _ok(self, code):
        if code:
            text = self._error_string(code).decode(errors="replace")
            raise RuntimeError(f"NCCL bootstrap failed: {text}")

    def integer(self, name, comm):
        out = ctypes.c_int(-1)
        self._ok(self._query[name](comm, ctypes.byref(out)))
        return out.value

    def all_gather_bytes(self, comm, send, recv, count, stream):
        self._ok(self._all_gather(send, recv, count, _NCCL_UINT8, comm, stream))

    def _point_to_point(self):
        if not hasattr(self, "_send"):
            void_p, c_int = ctypes.c_void_p, ctypes.c_int
            for attribute, name in (("_send", "ncclSend"), ("_recv", "ncclRecv")):
                fn = getattr(self._dso, name)
                fn.argtypes, fn.restype = [void_p, ctypes.c_size_t, c_int, c_int, void_p, void_p], c_int
                setattr(self, attribute, fn)
            for attribute, name in (("_group_start", "ncclGroupStart"), ("_group_end", "ncclGroupEnd")):
                fn = getattr(self._dso, name)
                fn.argtypes, fn.restype = [], c_int
                setattr(self, attribute, fn)

    def exchange_bytes(self, comm, sends, recvs, stream):
        """``sends`` / ``recvs``: (pointer, bytes, peer) triples, one NCCL group for all of them."""
        self._point_to_point()
        self._ok(self._group_start())
        try:
            for pointer, count, peer in sends:
                self._ok(self._send(pointer, count, _NCCL_UINT8, peer, comm, stream))
            for pointer, count, peer in recvs:
                self._ok(self._recv(pointer, count, _NCCL_UINT8, peer, comm, stream))
        finally:
            self._ok(self._group_end())


class NCCLCommHandle(ControlPlane):
    """A raw ``ncclComm_t`` plus the object that keeps it alive.

    Build one with :meth:`borrow` or :func:`get_nccl_comm_handle`. There is no
    destructor: shutdown order (close EP contexts, then destroy the group) is
    the application's job.
    """

    def __init__(self):
        raise TypeError("use NCCLCommHandle.borrow() or get_nccl_comm_handle()")

    @classmethod
    def borrow(cls, pointer, *, owner, library_path, group=None):
        """Wrap an existing communicator using its owner's NCCL library.

        ``group``, when given, must describe the same ordered ranks. The
        communicator must be in NCCL's normal blocking mode.
        """
        if isinstance(pointer, ctypes.c_void_p):
            pointer = pointer.value
        if isinstance(pointer, bool) or not isinstance(pointer, int) or pointer <= 0:
            raise ValueError("a non-null NCCL communicator pointer is required")
        if owner is None:
            raise ValueError("a borrowed communicator requires a lifetime owner")
        self = object.__new__(cls)
        self._owner = owner
        self._pointer = pointer
        self._api = _NcclApi(library_path)
        self.group = group
        self.rank = self._api.integer("ncclCommUserRank", pointer)
        self.world_size = self._api.integer("ncclCommCount", pointer)
        self.device = torch.device("cuda", self._api.integer("ncclCommCuDevice", pointer))
        if not 0 <= self.rank < self.world_size:
            raise ValueError("invalid NCCL communicator rank or size")
        if group is not None:
            self.validate_group(group)
        return self

    def get(self):
        """The borrowed raw pointer; no collective, no CUDA call."""
        return self._pointer

    def validate_group(self, group):
        if not dist.is_initialized():
            raise RuntimeError("initialize the supplied process group first")
        if (dist.get_rank(group), dist.get_world_size(group)) != (self.rank, self.world_size):
            raise ValueError("NCCL communicator and process group ranks do not match")
        if self.group is not None and self.group is not group and \
                dist.get_process_group_ranks(group) != dist.get_process_group_ranks(self.group):
            raise ValueError("NCCL communicator and process group membership do not match")

    def _gather(self, payload: torch.Tensor) -> torch.Tensor:
        # Both buffers are allocated on the current stream, so the upload above
        # and the caller's .cpu() below order themselves around the raw call.
        out = torch.empty((self.world_size, payload.numel()), dtype=torch.uint8, device=self.device)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        self._api.all_gather_bytes(self._pointer, payload.data_ptr(), out.data_ptr(), payload.numel(), stream)
        return out

    def all_gather_object(self, value):
        """Collective exchange of small trusted metadata (pickled).

        Setup/teardown only. Aggregate size is capped at 16 MiB. These raw
        collectives are not PyTorch ``Work`` objects, so no watchdog bounds them:
        the application bounds worker lifetime.
        """
        blob = pickle.dumps(value, protocol=pickle.HIGHEST_PROTOCOL)
        with torch.cuda.device(self.device):
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("NCCL bootstrap must finish before CUDA Graph capture")
            header = torch.frombuffer(bytearray(struct.pack("<q", len(blob))), dtype=torch.uint8).to(self.device)
            sizes = [struct.unpack("<q", bytes(row.tolist()))[0] for row in self._gather(header).cpu()]
            widest = max(sizes)
            if min(sizes) <= 0 or widest * self.world_size > _MAX_METADATA_BYTES:
                raise ValueError("NCCL bootstrap metadata exceeds the 16 MiB aggregate limit")
            staged = torch.zeros(widest, dtype=torch.uint8)
            staged[:len(blob)] = torch.frombuffer(bytearray(blob), dtype=torch.uint8)
            rows = self._gather(staged.to(self.device)).cpu()
        return [pickle.loads(rows[r, :sizes[r]].numpy().tobytes()) for r in range(self.world_size)]

    def exchange(self, send, recv):
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device)
            recv[self.rank].copy_(send[self.rank])
            sends = [(t.data_ptr(), t.numel() * t.element_size(), peer) for peer, t in enumerate(send)
                     if peer != self.rank and t.numel()]
            recvs = [(t.data_ptr(), t.numel() * t.element_size(), peer) for peer, t in enumerate(recv)
                     if peer != self.rank and t.numel()]
            for tensor in list(send) + list(recv):
                if not tensor.is_contiguous() or tensor.device != self.device:
                    raise ValueError("exchange needs contiguous tensors on the communicator's device")
            if sends or recvs:
                self._api.exchange_bytes(self._pointer, sends, recvs, stream.cuda_stream)

    def barrier(self):
        """Teardown rendezvous, outside the token data path."""
        with torch.cuda.device(self.device):
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("NCCL teardown cannot run during CUDA Graph capture")
            self._gather(torch.zeros(1, dtype=torch.uint8, device=self.device)).cpu()


_live_handles = weakref.WeakValueDictionary()
# Warm-up bookkeeping outlives handles: a handle garbage-collected on ONE rank
# must not make that rank's next lookup issue an unmatched collective.
_warmed = weakref.WeakKeyDictionary()


def get_nccl_comm_handle(group=None, device=None):
    """Borrow the communicator of a PyTorch NCCL process group.

    Collective on first use per (group, device): it makes PyTorch create its
    lazy communicator with one tiny all-reduce, then reads ``_comm_ptr()``.
    Call it before CUDA Graph capture.
    """
    if not dist.is_initialized():
        raise RuntimeError("initialize the NCCL process group first")
    group = dist.group.WORLD if group is None else group
    if str(dist.get_backend(group)) != "nccl":
        raise ValueError("get_nccl_comm_handle requires an NCCL process group")
    wanted = torch.cuda.current_device() if device is None else device
    wanted = torch.device("cuda", wanted) if isinstance(wanted, int) else torch.device(wanted)
    if wanted.type != "cuda":
        raise ValueError("NCCL communicator device must be CUDA")
    device = torch.device("cuda", torch.cuda.current_device() if wanted.index is None else wanted.index)
    key = (group, device)
    cached = _live_handles.get(key)
    if cached is not None:
        return cached
    backend = group._get_backend(device)
    if not callable(getattr(backend, "_comm_ptr", None)):
        raise RuntimeError("PyTorch does not expose _comm_ptr(); obtain an NCCLCommHandle.borrow() "
                           "from the framework before constructing Context")
    with torch.cuda.device(device):
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("obtain the NCCL communicator before CUDA Graph capture")
        if device not in _warmed.get(group, ()):
            dist.all_reduce(torch.zeros(1, device=device), group=group)
            torch.cuda.current_stream(device).synchronize()
            _warmed.setdefault(group, set()).add(device)
        library = Path(torch.__file__).resolve().parent / "lib" / "libtorch_cuda.so"
        handle = NCCLCommHandle.borrow(backend._comm_ptr(), owner=group, group=group, library_path=library)
    if handle.device != device:
        raise ValueError("the process group's NCCL communicator is bound to another CUDA device")
    _live_handles[key] = handle
    return handle
