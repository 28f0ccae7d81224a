"""The SGLang source-tree integrator on a miniature tree that has the anchored lines of the
audited revision, and the SGLang binding against stand-in framework modules (the reference tests
its adapter the same way, tests/test_adapter.py:59-145)."""

import importlib
import importlib.util
import os
import sys
import types

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_integrator():
    spec = importlib.util.spec_from_file_location("epx_sglang_integrate",
                                                  os.path.join(ROOT, "adapters", "sglang", "integrate.py"))
    module = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = module
    spec.loader.exec_module(module)
    return module


MINIATURE = {
    "layers/moe/utils.py": '''from enum import Enum


class MoeA2ABackend(Enum):
    NONE = "none"
    DEEPEP = "deepep"

    def is_none(self):
        return self == MoeA2ABackend.NONE

    def is_deepep(self):
        return self == MoeA2ABackend.DEEPEP

    def is_deepep_v2(self):
        return False


def get_moe_a2a_backend():
    return MoeA2ABackend.NONE


def is_deepep_class_backend() -> bool:
    b = get_moe_a2a_backend()
    return (
        b.is_deepep()
        or b.is_deepep_v2()
    )
''',
    "arg_groups/fields/exec_.py": '''from typing import Annotated as A, Literal


def arg(**kwargs):
    return kwargs


class Exec:
    moe_a2a_backend: A[
        Literal[
            "none",
            "deepep",
        ],
        arg(
            help="Choose the backend for MoE A2A.",
            choices=[
                "none",
                "deepep",
            ],
        ),
    ] = "none"
''',
    "arg_groups/overrides.py": '''_A2A_EP_SPANNING_BACKENDS = frozenset(
    {
        "deepep",
    }
)
''',
    "arg_groups/moe_hook.py": '''def handle(server_args, cfg):
    a2a_backend = resolved_view(server_args).moe_a2a_backend
    if cfg.enable_waterfill:
        pass
''',
    "layers/moe/fused_moe_triton/layer.py": '''def create_moe_dispatcher(
    moe_runner_config,
    quant_method,
) -> BaseDispatcher:
    a2a_backend = get_moe_a2a_backend()
    return None


class FusedMoE:
    def __init__(self, intermediate_size, reduce_results):
        self.moe_tp_size = 1
        self.intermediate_size_per_partition = intermediate_size // self.moe_tp_size
        self.reduce_results = reduce_results
''',
    "layers/moe/moe_runner/triton.py": '''def register_fused_func(a, b):
    return lambda f: f


@register_fused_func("none", "triton")
def fused_experts_none_to_triton(dispatch_output, quant_info, runner_config):
    return None
''',
    "model_executor/runner_backend/full_cuda_graph_backend.py": '''import torch


class FullCudaGraphBackend:
    def __init__(
        self,
        enable_memory_saver: bool = False,
        reuse_output_buffer: bool = False,
    ) -> None:
        self._graphs = {}

    def capture(self, shape_key):
        graph = torch.cuda.CUDAGraph()
        return graph

    def replay(self, shape_key):
        with graph_pool_replay_scope():
            self._graphs[shape_key].replay()
''',
    "utils/common.py": '''def require_mlp_sync(moe_a2a_backend):
        if moe_a2a_backend.is_deepep():
            return True
        elif moe_a2a_backend.is_none():
            return True
        return False
''',
}


@pytest.fixture
def tree(tmp_path):
    for relative, text in MINIATURE.items():
        path = tmp_path / "python" / "sglang" / "srt" / relative
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(text)
    return tmp_path


def snapshot(tree):
    return {str(p.relative_to(tree)): p.read_text() for p in sorted(tree.rglob("*.py"))}


def test_apply_is_exact_idempotent_and_reversible(tree, capsys):
    tool = load_integrator()
    before = snapshot(tree)
    assert tool.main([str(tree), "--check"]) == 0
    assert snapshot(tree) == before                                  # a dry run writes nothing
    assert tool.main([str(tree)]) == 0
    applied = snapshot(tree)
    assert set(applied) == set(before) and all(applied[p] != before[p] for p in before)
    for path, text in applied.items():
        compile(text, path, "exec")
        assert text.count(tool.BEGIN) == text.count(tool.END) >= 1
    utils = applied["python/sglang/srt/layers/moe/utils.py"]
    scope = {}
    exec(compile(utils, "utils.py", "exec"), scope)
    backend = scope["MoeA2ABackend"]("ep_xpress_b200")
    assert backend.is_ep_xpress_b200() and not backend.is_none()
    scope["get_moe_a2a_backend"] = lambda: backend
    assert scope["is_deepep_class_backend"]() is True                # combine happens inside the dispatcher
    assert '"ep_xpress_b200",' in applied["python/sglang/srt/arg_groups/fields/exec_.py"]
    assert applied["python/sglang/srt/arg_groups/fields/exec_.py"].count('"ep_xpress_b200",') == 2
    assert "B200EPDispatcher(moe_runner_config)" in applied["python/sglang/srt/layers/moe/fused_moe_triton/layer.py"]
    assert "run_experts" in applied["python/sglang/srt/layers/moe/moe_runner/triton.py"]
    graph = applied["python/sglang/srt/model_executor/runner_backend/full_cuda_graph_backend.py"]
    assert graph.index("prepare_graph_capture()") < graph.index("graph = torch.cuda.CUDAGraph()")
    assert graph.index("prepare_graph_replay()") < graph.index("self._graphs[shape_key].replay()")
    capsys.readouterr()
    assert tool.main([str(tree)]) == 0                               # second run: nothing to do
    assert "nothing to apply" in capsys.readouterr().out
    assert snapshot(tree) == applied
    assert tool.main([str(tree), "--reverse"]) == 0
    assert snapshot(tree) == before                                  # byte for byte


def test_a_missing_or_ambiguous_anchor_stops_before_any_write(tree):
    tool = load_integrator()
    common = tree / "python/sglang/srt/utils/common.py"
    common.write_text(common.read_text().replace("is_none", "is_nothing"))
    before = snapshot(tree)
    with pytest.raises(SystemExit, match="nothing was written"):
        tool.main([str(tree)])
    assert snapshot(tree) == before
    common.write_text(MINIATURE["utils/common.py"] * 2)               # the anchor twice
    before = snapshot(tree)
    with pytest.raises(SystemExit, match="occurs 2 times"):
        tool.main([str(tree)])
    assert snapshot(tree) == before


def test_a_hand_edited_tree_with_torn_markers_is_refused(tree):
    tool = load_integrator()
    tool.main([str(tree)])
    common = tree / "python/sglang/srt/utils/common.py"
    common.write_text(common.read_text().replace(tool.END, "# gone"))
    with pytest.raises(SystemExit, match="begin marker without an end marker"):
        tool.main([str(tree), "--reverse"])


# ---- the binding against stand-in framework modules ---------------------------------------------
class _Parallel:
    moe_ep_size = tp_size = attn_dp_size = 2
    moe_ep_rank = 1

    class moe_ep_group:
        device_group = "ep-group"


class _RunnerConfig:
    hidden_size, top_k, num_experts, num_local_experts, layer_id = 256, 2, 8, 4, 7
    params_dtype = torch.bfloat16
    num_fused_shared_experts = 0
    no_combine = apply_router_weight_on_input = use_tp_all_gather_activation = False
    activation, is_gated = "silu", True
    routed_scaling_factor = None


@pytest.fixture
def binding(monkeypatch):
    state = {"capacity": 48, "extend": False}

    def module(name, **members):
        mod = types.ModuleType(name)
        mod.__dict__.update(members)
        monkeypatch.setitem(sys.modules, name, mod)
        return mod

    class BaseDispatcher:
        def __init__(self):
            self.base_ready = True

    class DispatchOutputFormat:
        STANDARD = "standard"

    class StandardCombineInput:
        def __init__(self, hidden_states):
            self.hidden_states = hidden_states

    class StandardTopKOutput:
        def __init__(self, topk_weights, topk_ids, router_logits):
            self.topk_weights, self.topk_ids, self.router_logits = topk_weights, topk_ids, router_logits

    class TopKOutputChecker:
        @staticmethod
        def format_is_standard(output):
            return isinstance(output, StandardTopKOutput)

    for name in ("sglang", "sglang.srt", "sglang.srt.layers", "sglang.srt.layers.moe",
                 "sglang.srt.layers.moe.token_dispatcher"):
        module(name)
    module("sglang.srt.layers.dp_attention", get_global_dp_buffer_len=lambda: state["capacity"],
           get_is_extend_in_batch=lambda: state["extend"])
    module("sglang.srt.layers.moe.token_dispatcher.base", BaseDispatcher=BaseDispatcher,
           DispatchOutputFormat=DispatchOutputFormat)
    module("sglang.srt.layers.moe.token_dispatcher.standard", StandardCombineInput=StandardCombineInput)
    module("sglang.srt.layers.moe.topk", StandardTopKOutput=StandardTopKOutput, TopKOutputChecker=TopKOutputChecker)
    module("sglang.srt.runtime_context", get_parallel=lambda: _Parallel)
    monkeypatch.delitem(sys.modules, "ep_xpress_b200.adapters.sglang", raising=False)
    bound = importlib.import_module("ep_xpress_b200.adapters.sglang")
    fake_dist = types.SimpleNamespace(get_backend=lambda group: "nccl", get_world_size=lambda group: 2,
                                      get_rank=lambda group: 1)
    monkeypatch.setattr(bound, "dist", fake_dist)
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda device=None: "stream")
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)
    monkeypatch.setattr(bound, "_comm_handle",
                        lambda group, device: types.SimpleNamespace(device=device, world_size=2, rank=1))
    for name in [k for k in os.environ if k.startswith("EPX_")]:
        monkeypatch.delenv(name)
    from ep_xpress_b200.adapters import dispatcher as neutral
    neutral._contexts.clear()
    yield types.SimpleNamespace(module=bound, state=state, topk=StandardTopKOutput, combine_input=StandardCombineInput)
    neutral._contexts.clear()
    sys.modules.pop("ep_xpress_b200.adapters.sglang", None)


class _Count:
    """A device scalar: reading it on the host is the bug."""
    def __bool__(self):
        raise AssertionError("valid_count was read on the host")
    __int__ = __index__ = __bool__


class _Context:
    def __init__(self, comm, placement, config):
        self.world_size, self.effective_channels = comm.world_size, 8
        self.placement, self.config, self.calls, self.graph = list(placement), config, [], False

    def enable_cuda_graph(self):
        self.graph = True

    def create_workspace(self, capacity, tokens):
        return ("workspace", capacity, tokens)

    def dispatch_on_stream(self, x, ids, weights, **kwargs):
        self.calls.append(("dispatch", kwargs))
        rows = kwargs["recv_capacity"]
        return types.SimpleNamespace(hidden=torch.zeros(rows, 4), local_ids=torch.full((rows, 2), -1),
                                     weights=torch.zeros(rows, 2), valid_count=_Count(), handle=("handle", rows))

    def partial_buffer(self, handle):
        return ("partial plane of", handle)

    def combine_on_stream(self, partial, handle, **kwargs):
        self.calls.append(("combine", partial, handle, kwargs))
        return "combined"

    def close(self):
        pass


def test_binding_follows_the_framework_contract(binding, monkeypatch):
    monkeypatch.setenv("EPX_CUDA_GRAPH", "1")
    monkeypatch.setenv("EPX_MAX_TOKENS", "64")
    monkeypatch.setenv("EPX_DECODE_MAX_TOKENS", "32")
    layer = binding.module.B200EPDispatcher(_RunnerConfig, context_factory=_Context)
    assert layer.base_ready
    topk = binding.topk(torch.ones(5, 2), torch.zeros(5, 2, dtype=torch.int64), None)
    out = layer.dispatch(torch.zeros(5, 256, dtype=torch.bfloat16), topk)
    context = layer._inner.context
    assert context.graph and context.placement == [0, 0, 0, 0, 1, 1, 1, 1]
    kind, kwargs = context.calls[0]
    assert kind == "dispatch" and kwargs["recv_capacity"] == 48 and kwargs["stream"] == "stream"
    assert kwargs["workspace"] == ("workspace", 48, 5)                 # decode: a cached per-layer workspace
    assert out.format == "standard" and isinstance(out.valid_count, _Count)
    assert out.partial_out == ("partial plane of", ("handle", 48))
    assert out.topk_output.router_logits.shape == (48, 0)
    with pytest.raises(RuntimeError, match="outstanding"):
        layer.dispatch(torch.zeros(5, 256, dtype=torch.bfloat16), topk)
    with pytest.raises(RuntimeError, match="failed earlier"):          # a failure is sticky
        layer.combine(binding.combine_input("partial"))

    layer = binding.module.B200EPDispatcher(_RunnerConfig, context_factory=_Context)
    binding.state.update(capacity=64, extend=True)
    layer.dispatch(torch.zeros(5, 256, dtype=torch.bfloat16), topk)
    assert "workspace" not in layer._inner.context.calls[-1][1]        # prefill: no retained workspace
    assert layer.combine(binding.combine_input("partial")) == "combined"
    assert layer._inner.context.calls[-1][:3] == ("combine", "partial", ("handle", 64))
    with pytest.raises(TypeError):
        layer.combine("not a combine input")


def test_binding_rejects_layouts_it_does_not_serve(binding, monkeypatch):
    class Odd(_RunnerConfig):
        num_experts = 9
    with pytest.raises(ValueError, match="evenly"):
        binding.module.B200EPDispatcher(Odd, context_factory=_Context)

    class Shared(_RunnerConfig):
        num_fused_shared_experts = 1
    with pytest.raises(ValueError, match="shared"):
        binding.module.B200EPDispatcher(Shared, context_factory=_Context)
    monkeypatch.setenv("EPX_TRANSPORT", "host_ce")
    with pytest.raises(ValueError, match="device transport"):
        binding.module.B200EPDispatcher(_RunnerConfig, context_factory=_Context)
    monkeypatch.delenv("EPX_TRANSPORT")
    monkeypatch.setattr(binding.module, "dist", types.SimpleNamespace(
        get_backend=lambda group: "gloo", get_world_size=lambda group: 2, get_rank=lambda group: 1))
    with pytest.raises(ValueError, match="NCCL"):
        binding.module.B200EPDispatcher(_RunnerConfig, context_factory=_Context)


def test_runner_entry_handles_empty_ranks_and_requires_the_count(binding):
    empty = types.SimpleNamespace(hidden_states=torch.zeros(0, 256), valid_count=None, topk_output=None)
    result = binding.module.run_experts(empty, None, _RunnerConfig)
    assert result.hidden_states is empty.hidden_states                 # the matching combine still runs
    rows = types.SimpleNamespace(hidden_states=torch.zeros(3, 256), valid_count=None, topk_output=None)
    with pytest.raises(ValueError, match="valid_count"):
        binding.module.run_experts(rows, None, _RunnerConfig)

    class Scaled(_RunnerConfig):
        routed_scaling_factor = 2.5
    with pytest.raises(ValueError, match="routed_scaling_factor"):
        binding.module.run_experts(rows, None, Scaled)


def test_serving_argument_guard():
    from ep_xpress_b200.adapters import validate_serving_args
    good = dict(tp_size=8, dp_size=8, ep_size=8, enable_dp_attention=True, dtype="bfloat16")
    validate_serving_args(types.SimpleNamespace(**good), types.SimpleNamespace())
    for change, message in (({"dtype": "float16"}, "BF16"), ({"pp_size": 2}, "pipeline"), ({"nnodes": 2}, "one node"),
                            ({"dp_size": 4}, "equal"), ({"enable_eplb": True}, "enable_eplb"),
                            ({"quantization": "fp8"}, "quantised"), ({"enable_dp_attention": False}, "attention")):
        with pytest.raises(ValueError, match=message):
            validate_serving_args(types.SimpleNamespace(**{**good, **change}), types.SimpleNamespace())
    with pytest.raises(ValueError, match="shared experts"):
        validate_serving_args(types.SimpleNamespace(**good), types.SimpleNamespace(n_shared_experts=1))
