"""Serving-framework adapter: what sits between an inference engine and a ``Context``.

The reference ships this layer for one framework (SGLang v0.5.21: a dispatcher class,
server-argument guards, a source patch and shell presets; ep_xpress/adapters/*.py,
adapters/sglang/*). Here it is framework-neutral: the guards, the channel policy, the
environment-driven configuration and the per-layer workspace cache are plain Python with
no framework import, and ``EPDispatcher`` exposes the ``dispatch``/``combine`` pair plus
the CUDA-graph hooks an engine's MoE layer and graph runner call.
"""

from .dispatcher import DispatchOutput, EPDispatcher, close_contexts, prepare_graph_capture, prepare_graph_replay
from .env import PRESETS, channel_policy_from_env, config_from_env
from .guards import (contiguous_expert_map, receive_capacity_from_scheduler, select_active_channels,
                     validate_expert_runner, validate_moe_layer, validate_runner_config, validate_server_args,
                     validate_serving_args)

__all__ = ["DispatchOutput", "EPDispatcher", "PRESETS", "channel_policy_from_env", "close_contexts", "config_from_env",
           "contiguous_expert_map", "prepare_graph_capture", "prepare_graph_replay",
           "receive_capacity_from_scheduler", "select_active_channels", "validate_expert_runner", "validate_moe_layer",
           "validate_runner_config", "validate_server_args", "validate_serving_args"]
