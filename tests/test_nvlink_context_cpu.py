"""Host-side logic of the NVLink context without a GPU: a bare instance with a mocked runtime
and patched ``torch.cuda`` entry points (the technique of the reference's
tests/test_host_sm_context.py:175-243)."""

import contextlib
import threading
from types import SimpleNamespace
from unittest import mock

import pytest
import torch

from ep_xpress_b200 import Config
from ep_xpress_b200.context import RouteHandle
from ep_xpress_b200.parallel import nvlink
from ep_xpress_b200.parallel.core import Slot, SlotViews


class FakeStream:
    def __init__(self, name):
        self.name, self.waits, self.cuda_stream = name, [], 0
        self.device = torch.device("cpu")

    def wait_stream(self, other):
        self.waits.append(other.name)

    def wait_event(self, event):
        self.waits.append("event")

    def synchronize(self):
        pass


class FakeEvent:
    def record(self, stream):
        self.stream = stream

    def query(self):
        return True


def fake_slot(capacity, tokens, hidden=16, topk=2):
    z = torch.zeros
    views = SlotViews(hidden=z(capacity, hidden, dtype=torch.bfloat16), local_ids=z(capacity, topk, dtype=torch.int64),
                      weights=z(capacity, topk), inverse=z(capacity, 2, dtype=torch.int64),
                      partial=z(capacity, hidden, dtype=torch.bfloat16), count=z(1, dtype=torch.int32),
                      mask=z(tokens, dtype=torch.int64), dest_rows=z(tokens, 2, dtype=torch.int32),
                      send_counts=z(2, dtype=torch.int32), recv_counts=z(2, dtype=torch.int32),
                      output=z(tokens, hidden, dtype=torch.bfloat16))
    return Slot(capacity, tokens, [0], [views])


@pytest.fixture()
def ctx():
    cfg = Config(hidden_size=16, topk=2, max_tokens_per_rank=8, slots=2, max_pending_operations=2, channels=4)
    c = object.__new__(nvlink.NVLinkContext)
    c.config, c.rank, c.world_size = cfg, 0, 2
    c.device = torch.device("cpu")
    c._id, c._lock = "ctx", threading.RLock()
    c._failed, c._closed, c._counter, c._pending = None, False, 0, 0
    c._graph_enabled, c._capture_ready, c._last_stream = False, False, None
    c._pool, c._workspaces, c._profile = [], [], None
    c._max_receive_capacity = 16
    c.effective_channels = 4
    c._work_stream = FakeStream("work")
    core = mock.Mock()
    core.max_ctas = 100
    c._negotiated_ctas = 100
    core.pick_ctas.side_effect = lambda tokens, budget=None: budget
    core.create_slot.side_effect = lambda capacity, tokens, stream=None: fake_slot(capacity, tokens)
    c._core = core
    current = FakeStream("main")
    patches = [mock.patch.object(torch.cuda, "device", lambda d: contextlib.nullcontext()),
               mock.patch.object(torch.cuda, "current_stream", lambda d=None: current),
               mock.patch.object(torch.cuda, "is_current_stream_capturing", lambda: False),
               mock.patch.object(torch.cuda, "stream", lambda s: contextlib.nullcontext()),
               mock.patch.object(torch.cuda, "Event", FakeEvent),
               mock.patch.object(torch.Tensor, "record_stream", lambda self, s: None)]
    for p in patches:
        p.start()
    yield SimpleNamespace(ep=c, core=core, main=current)
    for p in patches:
        p.stop()


def inputs(tokens=4):
    return (torch.zeros(tokens, 16, dtype=torch.bfloat16), torch.zeros(tokens, 2, dtype=torch.int64),
            torch.zeros(tokens, 2))


def test_direct_dispatch_plumbs_arguments_and_emits_no_ticket(ctx):
    batch = ctx.ep.dispatch_on_stream(*inputs(), recv_capacity=12, active_channels=2, tag={"layer": 3})
    assert batch.hidden.shape == (12, 16) and batch.handle.received_count == 12 and batch.handle.active_channels == 2
    _, kwargs = ctx.core.dispatch.call_args
    assert kwargs["identity"] == 0                      # tags are not even hashed without diagnostics
    assert kwargs["ctas"] == 50                         # 2 of 4 channels -> half of the CTA budget
    assert ctx.ep._pending == 0
    out = ctx.ep.combine_on_stream(torch.zeros(12, 16, dtype=torch.bfloat16), batch.handle)
    assert out.shape == (4, 16) and batch.handle._consumed
    with pytest.raises(ValueError, match="already been consumed"):
        ctx.ep.combine_on_stream(torch.zeros(12, 16, dtype=torch.bfloat16), batch.handle)


def test_diagnostics_hashes_phase_tag_and_operation(ctx):
    object.__setattr__(ctx.ep.config, "diagnostics", True)
    batch = ctx.ep.dispatch_on_stream(*inputs(), tag="a")
    assert ctx.core.dispatch.call_args[1]["identity"] == nvlink.operation_identity("dispatch", "a")
    ctx.ep.combine_on_stream(torch.zeros(16, 16, dtype=torch.bfloat16), batch.handle, tag="a")
    assert ctx.core.combine.call_args[1]["identity"] == nvlink.operation_identity("combine", "a", batch.handle.operation)
    assert nvlink.operation_identity("dispatch", "a") != nvlink.operation_identity("dispatch", "b")


@pytest.mark.parametrize("kwargs,error,fragment", [
    (dict(active_channels=0), ValueError, "active_channels"),
    (dict(active_channels=5), ValueError, "active_channels"),
    (dict(active_channels=True), ValueError, "active_channels"),
    (dict(recv_capacity=17), ValueError, "rank capacity"),
    (dict(fused_combine=True), ValueError, "decode mailbox"),
])
def test_local_misuse_is_rejected_before_anything_is_submitted(ctx, kwargs, error, fragment):
    with pytest.raises(error, match=fragment):
        ctx.ep.dispatch_on_stream(*inputs(), **kwargs)
    assert ctx.core.dispatch.call_count == 0 and ctx.ep._counter == 0 and ctx.ep._failed is None


def test_input_validation(ctx):
    with pytest.raises(ValueError, match="token capacity"):
        ctx.ep.dispatch_on_stream(*inputs(9))
    x, ids, w = inputs()
    with pytest.raises(ValueError, match="inference tensors"):
        ctx.ep.dispatch_on_stream(x, ids, w.requires_grad_())
    with pytest.raises(ValueError, match="handle belongs to another context"):
        ctx.ep.combine_on_stream(x, RouteHandle("other", 1, None, 4, 16))
    batch = ctx.ep.dispatch_on_stream(*inputs())
    with pytest.raises(ValueError, match="already-weighted"):
        ctx.ep.combine_on_stream(x, batch.handle, weights_applied=False)
    with pytest.raises(ValueError, match="BF16"):
        ctx.ep.combine_on_stream(torch.zeros(4, 16), batch.handle)


def test_implicit_slots_bound_outstanding_handles(ctx):
    first = ctx.ep.dispatch_on_stream(*inputs())
    second = ctx.ep.dispatch_on_stream(*inputs())
    with pytest.raises(RuntimeError, match="slots"):
        ctx.ep.dispatch_on_stream(*inputs())
    ctx.ep.combine_on_stream(torch.zeros(16, 16, dtype=torch.bfloat16), second.handle)   # reverse order is legal
    ctx.ep.dispatch_on_stream(*inputs())
    assert ctx.core.create_slot.call_count == 2
    assert first.handle.operation == 1 and second.handle.operation == 2


def test_workspace_lifetime_state_machine(ctx):
    ws = ctx.ep.create_workspace(12, 4)
    with pytest.raises(ValueError, match="shape or fused combine mode"):
        ctx.ep.dispatch_async(*inputs(3), workspace=ws)
    other = object.__new__(nvlink.Workspace)
    other._context_id, other.recv_capacity, other.local_tokens, other.fused_combine = "someone else", 12, 4, False
    with pytest.raises(ValueError, match="another context"):
        ctx.ep.dispatch_async(*inputs(), workspace=other)
    ticket = ctx.ep.dispatch_async(*inputs(), workspace=ws)
    assert ctx.ep._pending == 1 and "main" in ctx.ep._work_stream.waits
    batch = ticket.wait()
    assert ctx.ep._pending == 0 and "event" in ctx.main.waits
    with pytest.raises(RuntimeError, match="previous workspace combine"):
        ctx.ep.dispatch_async(*inputs(), workspace=ws)
    combined = ctx.ep.combine_async(torch.zeros(12, 16, dtype=torch.bfloat16), batch.handle)
    with pytest.raises(RuntimeError, match="previous workspace combine"):       # combine not waited yet
        ctx.ep.dispatch_async(*inputs(), workspace=ws)
    out = combined.wait()
    assert out.data_ptr() == ws.output.data_ptr()                                # borrowed storage
    newer = ctx.ep.dispatch_async(*inputs(), workspace=ws)
    with pytest.raises(RuntimeError, match="expired"):
        ticket.wait()
    with pytest.raises(ValueError, match="timeout"):
        newer.wait(timeout=1.0)
    newer.wait()


def test_pending_operations_are_bounded(ctx):
    batch = ctx.ep.dispatch_async(*inputs()).wait()
    combined = ctx.ep.combine_async(torch.zeros(16, 16, dtype=torch.bfloat16), batch.handle)
    second = ctx.ep.dispatch_async(*inputs())
    with pytest.raises(RuntimeError, match="too many pending"):
        ctx.ep.dispatch_async(*inputs())
    combined.wait()
    second.wait()
    assert ctx.ep._pending == 0


def test_graph_lifecycle_guards(ctx):
    with pytest.raises(RuntimeError, match="enable_cuda_graph"):
        ctx.ep.prepare_graph_capture()
    object.__setattr__(ctx.ep.config, "diagnostics", True)
    with pytest.raises(RuntimeError, match="diagnostics"):
        ctx.ep.enable_cuda_graph()
    object.__setattr__(ctx.ep.config, "diagnostics", False)
    ctx.ep.enable_cuda_graph()
    ws = ctx.ep.create_workspace(12, 4)
    with mock.patch.object(torch.cuda, "is_current_stream_capturing", lambda: True):
        with pytest.raises(RuntimeError, match="prepare_graph_capture is required"):
            ctx.ep.dispatch_on_stream(*inputs(), workspace=ws)
    assert ctx.ep._failed is None                                   # misuse does not poison
    ctx.ep.prepare_graph_capture()
    with mock.patch.object(torch.cuda, "is_current_stream_capturing", lambda: True):
        with pytest.raises(RuntimeError, match="direct-stream"):
            ctx.ep.dispatch_async(*inputs(), workspace=ws)
        with pytest.raises(RuntimeError, match="warmed, retained workspace"):
            ctx.ep.dispatch_on_stream(*inputs(), workspace=ws)      # never used eagerly yet
        with pytest.raises(RuntimeError, match="warmed, retained workspace"):
            ctx.ep.dispatch_on_stream(*inputs())
    batch = ctx.ep.dispatch_on_stream(*inputs(), workspace=ws)
    ctx.ep.combine_on_stream(torch.zeros(12, 16, dtype=torch.bfloat16), batch.handle)
    with mock.patch.object(torch.cuda, "is_current_stream_capturing", lambda: True):
        captured = ctx.ep.dispatch_on_stream(*inputs(), workspace=ws)
        ctx.ep.combine_on_stream(torch.zeros(12, 16, dtype=torch.bfloat16), captured.handle)
    other = FakeStream("replay")
    ctx.ep.prepare_graph_replay(other)
    assert other.waits == ["main"]                                  # stream transition only, no host sync


def test_failed_and_closed_contexts_refuse_work(ctx):
    ctx.core.dispatch.side_effect = RuntimeError("launch failed")
    with pytest.raises(RuntimeError, match="launch failed"):
        ctx.ep.dispatch_on_stream(*inputs())
    with pytest.raises(RuntimeError, match="failed state"):
        ctx.ep.dispatch_on_stream(*inputs())
    ctx.ep._failed, ctx.ep._closed = None, True
    with pytest.raises(RuntimeError, match="closed"):
        ctx.ep.dispatch_on_stream(*inputs())


def test_device_status_surfaces_at_check(ctx):
    ctx.core.status.return_value = (2, 0x0100000000000000, 5, 4)
    with pytest.raises(RuntimeError, match="nvlink: receive capacity exceeded"):
        ctx.ep.check()
    with pytest.raises(RuntimeError, match="failed state"):
        ctx.ep.check()


def test_set_tuning_bounds_the_launch_width(ctx):
    ctx.ep.set_tuning(items_per_cta=4, max_ctas=40)
    assert ctx.core.items_per_cta == 4 and ctx.core.max_ctas == 40
    ctx.ep.dispatch_on_stream(*inputs(), active_channels=2)
    assert ctx.core.dispatch.call_args[1]["ctas"] == 20          # half of the lowered budget
    with pytest.raises(ValueError, match="within 1..100"):
        ctx.ep.set_tuning(max_ctas=101)                            # never above the negotiated width
    with pytest.raises(ValueError, match="positive"):
        ctx.ep.set_tuning(items_per_cta=0)
    assert ctx.core.max_ctas == 40 and ctx.ep._failed is None      # misuse does not poison the context


def test_profile_report_is_only_readable_at_a_completed_boundary(ctx):
    with pytest.raises(RuntimeError, match="no completed"):
        ctx.ep.read_combine_profile()
    ctx.ep._profile = object()                                     # a capture is running
    with pytest.raises(RuntimeError, match="completed boundary"):
        ctx.ep.read_combine_profile()
    ctx.ep._profile = None
    ctx.ep._last_profile = {"operations": []}
    assert ctx.ep.read_combine_profile() == {"operations": []}
