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
        """Wrap a communicator that somebody else created, resolving NCCL from THEIR library.

        ``owner`` is whatever keeps the communicator alive (a process group, a framework object);
        the handle holds a reference to it and never destroys anything. ``group``, when given,
        must be the torch.distributed group with the same ordered ranks. The communicator has to
        be in NCCL's blocking mode.
        """
        address = pointer.value if isinstance(pointer, ctypes.c_void_p) else pointer
        if type(address) is not int or address <= 0:
            raise ValueError("borrow() needs the non-null address of an ncclComm_t")
        if owner is None:
            raise ValueError("borrow() needs a lifetime owner: the object that keeps the communicator alive")
        handle = object.__new__(cls)
        handle._owner, handle._pointer, handle.group = owner, address, group
        handle._api = api = _NcclApi(library_path)
        rank, size = api.integer("ncclCommUserRank", address), api.integer("ncclCommCount", address)
        if size < 1 or rank < 0 or rank >= size:
            raise ValueError(f"invalid NCCL communicator: rank {rank} of {size}")
        handle.rank, handle.world_size = rank, size
        handle.device = torch.device("cuda", api.integer("ncclCommCuDevice", address))
        if group is not None:
            handle.validate_group(group)
        return handle

    def get(self):
        """The borrowed raw pointer; no collective, no CUDA call."""
        return self._pointer

    def validate_group(self, group):
        """``group`` must describe the ranks of this communicator, in the same order."""
        if not dist.is_initialized():
            raise RuntimeError("the process group given to the handle is not initialised")
        described = (dist.get_rank(group), dist.get_world_size(group))
        if described != (self.rank, self.world_size):
            raise ValueError(f"the process group says rank {described[0]} of {described[1]}, the communicator "
                             f"rank {self.rank} of {self.world_size}")
        known = self.group
        if known is not None and known is not group:
            if dist.get_process_group_ranks(group) != dist.get_process_group_ranks(known):
                raise ValueError("the process group has other members than the communicator's own group")

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


def _cuda_device(device):
    """``None`` / index / ``"cuda"`` / ``"cuda:N"`` -> a fully indexed CUDA device."""
    if device is None:
        return torch.device("cuda", torch.cuda.current_device())
    chosen = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
    if chosen.type != "cuda":
        raise ValueError(f"an NCCL communicator lives on a CUDA device, not on {chosen}")
    return chosen if chosen.index is not None else torch.device("cuda", torch.cuda.current_device())


def get_nccl_comm_handle(group=None, device=None):
    """Borrow the communicator PyTorch built for an NCCL process group.

    PyTorch creates that communicator lazily, so the first call per (group, device) runs one
    tiny all-reduce - a collective: call it on every rank, and before any CUDA Graph capture.
    Later calls return the cached handle without communicating, also after the handle object
    was garbage-collected on some ranks only.
    """
    if not dist.is_initialized():
        raise RuntimeError("initialize the NCCL process group first")
    group = group if group is not None else dist.group.WORLD
    backend_name = str(dist.get_backend(group))
    if backend_name != "nccl":
        raise ValueError(f"the group's backend is {backend_name}; only an NCCL group has a communicator to borrow")
    device = _cuda_device(device)
    handle = _live_handles.get((group, device))
    if handle is not None:
        return handle
    backend = group._get_backend(device)
    pointer_of = getattr(backend, "_comm_ptr", None)
    if not callable(pointer_of):
        raise RuntimeError("this PyTorch build has no ProcessGroupNCCL._comm_ptr(); get the raw communicator from "
                           "your framework and pass it to NCCLCommHandle.borrow()")
    with torch.cuda.device(device):
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("get_nccl_comm_handle() communicates: call it before CUDA Graph capture starts")
        warmed = _warmed.setdefault(group, set())
        if device not in warmed:
            dist.all_reduce(torch.zeros(1, device=device), group=group)
            torch.cuda.current_stream(device).synchronize()
            warmed.add(device)
        torch_nccl = Path(torch.__file__).resolve().parent / "lib" / "libtorch_cuda.so"
        handle = NCCLCommHandle.borrow(pointer_of(), owner=group, group=group, library_path=torch_nccl)
    if handle.device != device:
        raise ValueError(f"the group's communicator belongs to {handle.device}, not to {device}")
    _live_handles[(group, device)] = handle
    return handle
