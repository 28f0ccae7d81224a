"""SGLang binding: a token dispatcher and an expert runner for the ``ep_xpress_b200`` A2A backend.

Importing this module imports SGLang. ``adapters/sglang/integrate.py`` (repository root) makes
an SGLang source tree name the backend and call the entry points below; nothing else of the
library knows SGLang. What the reference does with ``HostEPDispatcher`` plus a Triton-runner
patch (ep_xpress/adapters/sglang.py:91-340, ep_xpress/adapters/sglang_valid.py,
adapters/sglang/sglang-v0.5.21.patch) is here:

* ``B200EPDispatcher`` - SGLang's ``BaseDispatcher`` contract over the framework-neutral
  ``EPDispatcher``: one shared ``Context`` per (group, device, config, placement), per-layer
  decode workspaces, the scheduler's padded token sum as receive capacity, one outstanding
  operation per layer, everything on the caller's stream (so eager steps and full decode CUDA
  graphs take the same path), the device-side ``valid_count`` handed to the runner.
* ``run_experts`` - the count-aware BF16 expert runner registered for (this backend, the
  ``triton`` runner slot): the tcgen05 grouped SwiGLU of ``ops.GroupedSwiGLU`` writes weighted
  partial rows straight into the combine's partial plane. SGLang's own Triton kernels are not
  patched and not used for routed experts.
* ``prepare_graph_capture`` / ``prepare_graph_replay`` / ``close_contexts`` - the hooks of the
  full-graph runner and of shutdown.
"""

from __future__ import annotations

import logging
import os
from typing import NamedTuple

import torch
import torch.distributed as dist

from sglang.srt.layers.dp_attention import get_global_dp_buffer_len, get_is_extend_in_batch
from sglang.srt.layers.moe.token_dispatcher.base import BaseDispatcher, DispatchOutputFormat
from sglang.srt.layers.moe.token_dispatcher.standard import StandardCombineInput
from sglang.srt.layers.moe.topk import StandardTopKOutput, TopKOutputChecker
from sglang.srt.runtime_context import get_parallel

from .dispatcher import EPDispatcher, close_contexts, prepare_graph_capture, prepare_graph_replay
from .env import channel_policy_from_env, config_from_env
from .guards import contiguous_expert_map, validate_moe_layer

BACKEND = "ep_xpress_b200"
log = logging.getLogger(__name__)

__all__ = ["BACKEND", "B200EPDispatcher", "CountedDispatchOutput", "close_contexts", "prepare_graph_capture",
           "prepare_graph_replay", "release_runners", "run_experts"]


class CountedDispatchOutput(NamedTuple):
    """SGLang's standard expert input plus what only this backend has: the number of valid rows
    as a DEVICE scalar and the plane the runner should write its weighted rows to."""
    hidden_states: object
    hidden_states_scale: object
    topk_output: object
    valid_count: object
    partial_out: object = None
    hidden_states_pre_quant: object = None

    @property
    def format(self):
        return DispatchOutputFormat.STANDARD


def _flag(name, default):
    text = os.environ.get(name, default)
    if text not in ("0", "1"):
        raise ValueError(f"{name} must be 0 or 1")
    return text == "1"


def _comm_handle(group, device):
    """The EP group's own NCCL communicator (collective on first use: before any graph capture)."""
    from ..comm import get_nccl_comm_handle
    return get_nccl_comm_handle(group, device=device)


class B200EPDispatcher(BaseDispatcher):
    """One per MoE layer. SGLang's combine input carries no handle, so a layer has exactly one
    operation outstanding: dispatch, experts, combine, in that order, on every EP rank -
    also on ranks with no tokens of their own or none to receive."""

    def __init__(self, moe_runner_config, *, context_factory=None):
        super().__init__()
        parallel = get_parallel()
        size = parallel.moe_ep_size
        if not (parallel.tp_size == parallel.attn_dp_size == size):
            raise ValueError("attention DP size, TP size and EP size must be equal")
        validate_moe_layer(moe_runner_config, world_size=size, bf16=torch.bfloat16)
        self._group = parallel.moe_ep_group.device_group
        if str(dist.get_backend(self._group)) != "nccl":
            raise ValueError("the EP group must be an NCCL group: its communicator carries the bootstrap")
        if dist.get_world_size(self._group) != size or dist.get_rank(self._group) != parallel.moe_ep_rank:
            raise ValueError("the EP device group does not match the framework's EP size and rank order")
        self._device = torch.device("cuda", torch.cuda.current_device())
        self._graphs = _flag("EPX_CUDA_GRAPH", "0")
        self._config = config_from_env(moe_runner_config.hidden_size, moe_runner_config.top_k,
                                       int(os.environ.get("EPX_MAX_TOKENS", "16384")))
        if not self._config.device_transport:
            raise ValueError("the SGLang binding serves the device transport (EPX_TRANSPORT=nvlink)")
        self._policy = channel_policy_from_env()
        self._placement = tuple(contiguous_expert_map(moe_runner_config.num_experts, size))
        self._layer_id = moe_runner_config.layer_id
        self._factory = context_factory
        self._inner = None
        self._failed = False

    def _dispatcher(self):
        """Created on the first forward: the context allocates and exchanges memory handles, which
        must neither happen while weights load nor inside a capture."""
        if self._inner is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("run one eager forward before capturing: the EP context is created on first use")
            self._inner = EPDispatcher(_comm_handle(self._group, self._device), self._placement, self._config,
                                       layer_id=self._layer_id, group_key=self._group,
                                       context_factory=self._factory, enable_cuda_graph=self._graphs,
                                       channel_policy=self._policy)
        return self._inner

    def _alive(self):
        if self._failed:
            raise RuntimeError("this EP dispatcher failed earlier; restart the worker group")

    def dispatch(self, hidden_states, topk_output):
        self._alive()
        if not TopKOutputChecker.format_is_standard(topk_output):
            raise ValueError("the EP dispatcher needs standard top-k ids and weights")
        try:
            inner = self._dispatcher()
            stream = torch.cuda.current_stream(self._device)
            # The padded sum of every rank's scheduled tokens, known on the host before the forward:
            # a token reaches a rank at most once, so it bounds the received rows whatever top-k is.
            out = inner.dispatch(hidden_states, topk_output.topk_ids, topk_output.topk_weights,
                                 recv_capacity=get_global_dp_buffer_len(),
                                 is_decode=not get_is_extend_in_batch(), stream=stream)
            rows = out.hidden_states.shape[0]
            partial_buffer = getattr(inner.context, "partial_buffer", None)
            return CountedDispatchOutput(
                hidden_states=out.hidden_states, hidden_states_scale=None,
                topk_output=StandardTopKOutput(
                    topk_weights=out.weights, topk_ids=out.local_expert_ids,
                    router_logits=out.hidden_states.new_empty((rows, 0), dtype=torch.float32)),
                valid_count=out.valid_count,
                partial_out=partial_buffer(out.handle) if partial_buffer is not None else None)
        except Exception:
            self._failed = True
            raise

    def combine(self, combine_input):
        self._alive()
        if not isinstance(combine_input, StandardCombineInput):
            raise TypeError("the EP dispatcher combines a StandardCombineInput")
        if self._inner is None:
            raise RuntimeError("combine needs a matching dispatch")
        try:
            return self._inner.combine(combine_input.hidden_states,
                                       stream=torch.cuda.current_stream(self._device))
        except Exception:
            self._failed = True
            raise


# ---- expert runner -----------------------------------------------------------------------------
_runners = {}


def _runner_for(w13, w2, rows, topk):
    """One grouped-GEMM runner per (layer weights, row bound); its scratch planes are allocated
    once, outside any capture (warm every graph bucket eagerly first, as for the workspaces)."""
    from ..ops.moe import GroupedSwiGLU
    key = (w13.data_ptr(), w2.data_ptr(), topk)
    runner = _runners.get(key)
    if runner is None or runner.max_rows < rows:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("warm each graph bucket before capture: the expert runner allocates its planes")
        bound = max(rows, runner.max_rows if runner is not None else 0)
        runner = GroupedSwiGLU(w13, w2, max_rows=bound, topk=topk, pair_ctas=_flag("EPX_GEMM_CTA_PAIRS", "1"))
        _runners[key] = runner
    return runner


def run_experts(dispatch_output, quant_info, runner_config):
    """(ep_xpress_b200, triton) entry of SGLang's fused-expert registry: gated-SiLU experts over
    the first ``valid_count`` rows (a device scalar - never read on the host), each row's local
    slots weighted and summed in slot order with one rounding, the contract of the reference's
    runner (ep_xpress/adapters/sglang_valid.py:206-222). Rows at and beyond ``valid_count`` are
    not touched. A rank that received nothing still returns its (empty) input so that the
    matching combine runs."""
    hidden = dispatch_output.hidden_states
    if hidden.shape[0] == 0:
        return StandardCombineInput(hidden_states=hidden)
    if getattr(runner_config, "routed_scaling_factor", None) not in (None, 1.0):
        raise ValueError("routed_scaling_factor must be folded into the router weights for this runner")
    valid_count = getattr(dispatch_output, "valid_count", None)
    if valid_count is None:
        raise ValueError("the expert runner needs the dispatcher's device-side valid_count")
    topk = dispatch_output.topk_output
    runner = _runner_for(quant_info.w13_weight, quant_info.w2_weight, hidden.shape[0], topk.topk_ids.shape[1])
    out = runner(hidden, topk.topk_ids, topk.topk_weights, valid_count, out=getattr(dispatch_output, "partial_out", None))
    return StandardCombineInput(hidden_states=out)


def release_runners():
    """Drop the cached expert runners (their scratch planes); call between model reloads."""
    _runners.clear()
