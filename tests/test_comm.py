"""Borrowed-communicator handle with a mocked NCCL library (no GPU, no NCCL)."""

import ctypes
from unittest import mock

import pytest

from ep_xpress_b200 import Config, Context, NCCLCommHandle
from ep_xpress_b200 import comm as comm_module


class FakeApi:
    def __init__(self, path):
        self.path = path

    def integer(self, name, pointer):
        return {"ncclCommUserRank": 1, "ncclCommCount": 4, "ncclCommCuDevice": 0}[name]


def test_borrow_validates_pointer_and_owner():
    with mock.patch.object(comm_module, "_NcclApi", FakeApi):
        with pytest.raises(ValueError, match="non-null"):
            NCCLCommHandle.borrow(0, owner=object(), library_path="x")
        with pytest.raises(ValueError, match="non-null"):
            NCCLCommHandle.borrow(True, owner=object(), library_path="x")
        with pytest.raises(ValueError, match="lifetime owner"):
            NCCLCommHandle.borrow(1234, owner=None, library_path="x")
        owner = object()
        handle = NCCLCommHandle.borrow(ctypes.c_void_p(1234), owner=owner, library_path="lib.so")
        assert (handle.rank, handle.world_size, handle.get()) == (1, 4, 1234)
        assert handle._owner is owner and str(handle.device) == "cuda:0"


def test_handles_are_not_constructed_directly_and_contexts_reject_raw_pointers():
    with pytest.raises(TypeError, match="borrow"):
        NCCLCommHandle()
    cfg = Config(hidden_size=64, topk=2, max_tokens_per_rank=8)
    with pytest.raises(TypeError, match="NCCLCommHandle"):
        Context(42, [0, 1], cfg)
    with pytest.raises(TypeError):
        Context(42, [0, 1], cfg, bootstrap_group=None)        # removed keyword of older releases
    with pytest.raises(TypeError, match="Config"):
        Context(42, [0, 1], {"hidden_size": 64})


def test_get_handle_requires_an_initialised_nccl_group():
    with pytest.raises(RuntimeError, match="initialize the NCCL process group"):
        comm_module.get_nccl_comm_handle(None)


def test_invalid_rank_from_the_library_is_rejected():
    class Broken(FakeApi):
        def integer(self, name, pointer):
            return {"ncclCommUserRank": 5, "ncclCommCount": 4, "ncclCommCuDevice": 0}[name]
    with mock.patch.object(comm_module, "_NcclApi", Broken):
        with pytest.raises(ValueError, match="invalid NCCL communicator"):
            NCCLCommHandle.borrow(99, owner=object(), library_path="x")


class FakeFunction:
    def __init__(self, log, name, result=0):
        self.log, self.name, self.result = log, name, result
        self.argtypes, self.restype = None, None

    def __call__(self, *args):
        self.log.append((self.name,) + args)
        return self.result


def test_point_to_point_exchange_is_one_nccl_group():
    log = []
    api = object.__new__(comm_module._NcclApi)
    api._dso = type("Dso", (), {name: FakeFunction(log, name) for name in
                                ("ncclSend", "ncclRecv", "ncclGroupStart", "ncclGroupEnd")})()
    api._error_string = lambda code: b"boom"
    api.exchange_bytes(77, sends=[(1000, 16, 2), (2000, 32, 3)], recvs=[(3000, 8, 2)], stream=5)
    assert [entry[0] for entry in log] == ["ncclGroupStart", "ncclSend", "ncclSend", "ncclRecv", "ncclGroupEnd"]
    assert log[1] == ("ncclSend", 1000, 16, 1, 2, 77, 5)          # bytes as ncclUint8, to peer 2
    assert log[3] == ("ncclRecv", 3000, 8, 1, 2, 77, 5)
    # a failing call still closes the group, then raises
    log.clear()
    api._dso.ncclRecv.result = 3
    with pytest.raises(RuntimeError, match="boom"):
        api.exchange_bytes(77, sends=[], recvs=[(3000, 8, 2)], stream=5)
    assert log[-1][0] == "ncclGroupEnd"


def test_get_handle_warms_up_once_and_caches(monkeypatch):
    import contextlib
    import torch
    import torch.distributed as dist

    class Backend:
        def _comm_ptr(self):
            return 4321

    class Group:
        def _get_backend(self, device):
            return Backend()

    group, reductions = Group(), []
    monkeypatch.setattr(comm_module, "_NcclApi", FakeApi)
    monkeypatch.setattr(dist, "is_initialized", lambda: True)
    monkeypatch.setattr(dist, "get_backend", lambda g: "nccl")
    monkeypatch.setattr(dist, "get_rank", lambda g=None: 1)
    monkeypatch.setattr(dist, "get_world_size", lambda g=None: 4)
    monkeypatch.setattr(dist, "all_reduce", lambda tensor, group=None: reductions.append(group))
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    monkeypatch.setattr(torch.cuda, "device", lambda d: contextlib.nullcontext())
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda d=None: mock.Mock())
    monkeypatch.setattr(torch, "zeros", lambda *shape, device=None: None)
    handle = comm_module.get_nccl_comm_handle(group)
    assert (handle.rank, handle.world_size, handle.get(), str(handle.device)) == (1, 4, 4321, "cuda:0")
    assert handle._owner is group and reductions == [group]
    assert comm_module.get_nccl_comm_handle(group, device="cuda") is handle and reductions == [group]
    del handle                                               # collected here, maybe not on other ranks:
    again = comm_module.get_nccl_comm_handle(group, 0)       # a new handle, but no second collective
    assert again.get() == 4321 and reductions == [group]
    with pytest.raises(ValueError, match="CUDA device"):
        comm_module.get_nccl_comm_handle(group, "cpu")
    monkeypatch.setattr(dist, "get_backend", lambda g: "gloo")
    with pytest.raises(ValueError, match="only an NCCL group"):
        comm_module.get_nccl_comm_handle(Group())
    monkeypatch.setattr(dist, "get_backend", lambda g: "nccl")
    monkeypatch.setattr(dist, "get_rank", lambda g=None: 0)
    with pytest.raises(ValueError, match="process group says rank 0 of 4"):
        comm_module.get_nccl_comm_handle(Group())
