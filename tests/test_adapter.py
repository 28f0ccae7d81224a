"""Adapter contract on CPU with a fake context (the reference tests its adapter against fake
framework modules, tests/test_adapter.py:59-145)."""

import pytest

from ep_xpress_b200 import Config
from ep_xpress_b200 import adapters
from ep_xpress_b200.adapters import dispatcher as dispatcher_module


class DeviceCount:
    """Stands for a CUDA int32[1]: touching it on the host is the bug the adapter must not have."""
    def __bool__(self):
        raise AssertionError("valid_count was read on the host")
    __int__ = __index__ = __bool__


class FakeTensor:
    def __init__(self, rows):
        self.shape = (rows, 8)


class FakeBatch:
    def __init__(self, handle):
        self.hidden, self.local_ids, self.weights = "hidden", "ids", "weights"
        self.valid_count, self.handle = DeviceCount(), handle


class FakeContext:
    created = 0

    def __init__(self, comm, placement, config):
        FakeContext.created += 1
        self.effective_channels = min(config.channels, 32)
        self.calls, self.workspaces, self.released, self.closed = [], [], [], False
        self._graph_enabled = False

    def enable_cuda_graph(self):
        self._graph_enabled = True

    def create_workspace(self, capacity, tokens):
        self.workspaces.append((capacity, tokens))
        return ("ws", capacity, tokens)

    def release_workspace(self, workspace):
        self.released.append(workspace)

    def dispatch_on_stream(self, x, ids, w, **kwargs):
        self.calls.append(("dispatch", kwargs))
        return FakeBatch(object())

    def combine_on_stream(self, partial, handle, **kwargs):
        self.calls.append(("combine", kwargs))
        return "out"

    def prepare_graph_capture(self):
        self.calls.append(("capture", {}))

    def prepare_graph_replay(self, stream=None):
        self.calls.append(("replay", {}))

    def close(self):
        self.closed = True


@pytest.fixture(autouse=True)
def fresh_registry():
    dispatcher_module._contexts.clear()
    FakeContext.created = 0
    yield
    dispatcher_module._contexts.clear()


def make(layer, cfg, comm="comm"):
    return adapters.EPDispatcher(comm, [0, 0, 1, 1], cfg, layer_id=layer, group_key="g", context_factory=FakeContext)


def test_layers_share_one_context_and_cache_workspaces():
    cfg = Config(hidden_size=64, topk=2, max_tokens_per_rank=64, decode_max_tokens=32, channels=8)
    a, b = make(0, cfg), make(1, cfg)
    assert a.context is b.context and FakeContext.created == 1
    out = a.dispatch(FakeTensor(16), None, None, token_counts=[16, 12], is_decode=True)
    assert isinstance(out.valid_count, DeviceCount)               # passed through untouched
    kind, kwargs = a.context.calls[-1]
    assert kind == "dispatch" and kwargs["recv_capacity"] == 28 and kwargs["active_channels"] == 2
    assert kwargs["workspace"] == ("ws", 28, 16) and kwargs["tag"] == ("layer", 0)
    with pytest.raises(RuntimeError, match="outstanding"):
        a.dispatch(FakeTensor(16), None, None, token_counts=[16, 12], is_decode=True)
    assert a.combine("partial") == "out"
    with pytest.raises(RuntimeError, match="no dispatched"):
        a.combine("partial")
    a.dispatch(FakeTensor(16), None, None, token_counts=[16, 12], is_decode=True)
    a.combine("partial")
    assert a.context.workspaces == [(28, 16)]                     # reused, not re-created
    for n in (1, 2, 3, 4):                                        # FIFO of four per layer
        a.dispatch(FakeTensor(n), None, None, token_counts=[n, n], is_decode=True)
        a.combine("p")
    assert a.context.released == [("ws", 28, 16)]


def test_prefill_uses_no_workspace_and_all_channels():
    cfg = Config(hidden_size=64, topk=2, max_tokens_per_rank=4096, channels=8)
    d = make(0, cfg)
    d.dispatch(FakeTensor(4096), None, None, token_counts=[4096, 100], is_decode=False)
    _, kwargs = d.context.calls[-1]
    assert "workspace" not in kwargs and kwargs["active_channels"] == 8 and kwargs["recv_capacity"] == 4196


def test_graph_hooks_and_teardown_reach_every_context():
    cfg = Config(hidden_size=64, topk=2, max_tokens_per_rank=64)
    d = make(0, cfg)
    e = adapters.EPDispatcher("other", [0, 1], cfg, layer_id=0, group_key="h", context_factory=FakeContext,
                              enable_cuda_graph=True)
    assert e.context._graph_enabled and not d.context._graph_enabled
    adapters.prepare_graph_capture()
    adapters.prepare_graph_replay()
    assert ("capture", {}) in d.context.calls and ("replay", {}) in e.context.calls
    adapters.close_contexts()
    assert d.context.closed and e.context.closed and not dispatcher_module._contexts


def test_guards():
    adapters.validate_server_args(tp_size=8, dp_size=8, ep_size=8)
    for bad in (dict(tp_size=8, dp_size=4, ep_size=8), dict(tp_size=8, dp_size=8, ep_size=8, pp_size=2),
                dict(tp_size=8, dp_size=8, ep_size=8, moe_tp_size=2),
                dict(tp_size=8, dp_size=8, ep_size=8, enable_dp_attention=False)):
        with pytest.raises(ValueError):
            adapters.validate_server_args(**bad)
    adapters.validate_runner_config(reduce_results=False)
    with pytest.raises(ValueError, match="reduce_results"):
        adapters.validate_runner_config(reduce_results=True)
    assert adapters.contiguous_expert_map(8, 4) == [0, 0, 1, 1, 2, 2, 3, 3]
    with pytest.raises(ValueError):
        adapters.contiguous_expert_map(9, 4)
    assert adapters.receive_capacity_from_scheduler([3, 0, 5], 8) == 8
    with pytest.raises(ValueError):
        adapters.receive_capacity_from_scheduler([9], 8)
    assert adapters.select_active_channels(1, 8, is_decode=True) == 1
    assert adapters.select_active_channels(33, 8, is_decode=True) == 5
    assert adapters.select_active_channels(3, 8, is_decode=False) == 3
    assert adapters.select_active_channels(4096, 8, is_decode=False) == 8
    assert adapters.select_active_channels(0, 8, is_decode=True) == 1


def test_config_from_env_precedence_and_validation():
    cfg = adapters.config_from_env(64, 2, 16, env={"EPX_PRESET": "b200_decode", "EPX_SLOTS": "3"}, channels=6)
    assert (cfg.transport, cfg.decode_max_tokens, cfg.slots, cfg.channels) == ("nvlink", 256, 3, 6)
    assert adapters.config_from_env(64, 2, 16, env={"EPX_DIAGNOSTICS": "true"}).diagnostics is True
    with pytest.raises(ValueError, match="unknown configuration"):
        adapters.config_from_env(64, 2, 16, env={"EPX_SLOT": "3"})
    with pytest.raises(ValueError, match="not a valid value"):
        adapters.config_from_env(64, 2, 16, env={"EPX_SLOTS": "many"})
    with pytest.raises(ValueError, match="unknown preset"):
        adapters.config_from_env(64, 2, 16, env={}, preset="h100")
    with pytest.raises(ValueError, match="channels"):
        adapters.config_from_env(64, 2, 16, env={"EPX_CHANNELS": "64"})


def test_channel_overrides_and_fixed_width():
    pick = adapters.select_active_channels
    assert pick(4096, 8, is_decode=False, prefill_override=3) == 3
    assert pick(4, 8, is_decode=True, decode_override=32) == 8           # clamped to what was allocated
    assert pick(4, 8, is_decode=True, prefill_override=3) == 1           # the other phase's override is ignored
    assert pick(1, 8, is_decode=True, adaptive=False) == 8
    with pytest.raises(ValueError, match="decode_override"):
        pick(4, 8, is_decode=True, decode_override=-1)
    with pytest.raises(ValueError, match="prefill_override"):
        pick(4, 8, is_decode=False, prefill_override=True)


def test_expert_runner_scope():
    adapters.validate_expert_runner()
    with pytest.raises(ValueError, match="gated SiLU"):
        adapters.validate_expert_runner(activation="gelu")
    with pytest.raises(ValueError, match="gated SiLU"):
        adapters.validate_expert_runner(is_gated=False)
    with pytest.raises(ValueError, match="activation modifiers"):
        adapters.validate_expert_runner(swiglu_limit=7.0)


def test_channel_policy_from_environment():
    env = {"EPX_ADAPTIVE_CHANNELS": "0", "EPX_DECODE_CHANNELS": "2", "EPX_COMBINE_STREAMING": "on"}
    policy = adapters.channel_policy_from_env(env)
    assert policy == {"adaptive": False, "decode_override": 2}
    cfg = adapters.config_from_env(64, 2, 8, env=env)                  # policy variables are not unknown
    assert cfg.combine_streaming == "on"
    assert adapters.select_active_channels(100, 8, is_decode=True, **policy) == 2
    assert adapters.select_active_channels(100, 8, is_decode=False, **policy) == 8
    with pytest.raises(ValueError, match="EPX_DECODE_TOKENS_PER_CHANNEL"):
        adapters.channel_policy_from_env({"EPX_DECODE_TOKENS_PER_CHANNEL": "0"})
    with pytest.raises(ValueError, match="not a valid value"):
        adapters.channel_policy_from_env({"EPX_PREFILL_CHANNELS": "many"})
