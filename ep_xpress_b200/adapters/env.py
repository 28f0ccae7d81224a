"""Runtime configuration from ``EPX_*`` environment variables, and named presets.

Replaces the reference adapter's ~25 ``EP_XPRESS_*`` runtime variables and chained shell
presets (ep_xpress/adapters/sglang.py:107-176, adapters/sglang/presets/*.sh). There is no
build-time tier: every knob below is a ``Config`` field.
"""

from __future__ import annotations

import os

from ..config import Config

_FIELDS = {
    "EPX_TRANSPORT": ("transport", str),
    "EPX_CHANNELS": ("channels", int),
    "EPX_SLOTS": ("slots", int),
    "EPX_TIMEOUT_SECONDS": ("timeout_seconds", float),
    "EPX_MAX_PENDING": ("max_pending_operations", int),
    "EPX_DECODE_MAX_TOKENS": ("decode_max_tokens", int),
    "EPX_DIAGNOSTICS": ("diagnostics", "bool"),
    "EPX_ZERO_PADDING": ("zero_padding", "bool"),
    "EPX_COMBINE_ROUNDING": ("combine_rounding", str),
    "EPX_GPU_POOL_BUDGET_BYTES": ("gpu_pool_budget_bytes", int),
    "EPX_WORKSPACE_POOL_BYTES": ("workspace_pool_bytes", int),
    "EPX_COOPERATIVE_LAUNCH": ("cooperative_launch", "bool"),
    "EPX_COMBINE_STREAMING": ("combine_streaming", str),
}

# Per-operation launch width of the dispatcher (not Config fields: they never change what is
# allocated). Counterparts of the reference's adaptive / prefill / decode channel variables
# (ep_xpress/adapters/sglang.py:107-176).
_POLICY = {
    "EPX_ADAPTIVE_CHANNELS": ("adaptive", "bool"),
    "EPX_PREFILL_CHANNELS": ("prefill_override", int),
    "EPX_DECODE_CHANNELS": ("decode_override", int),
    "EPX_DECODE_TOKENS_PER_CHANNEL": ("tokens_per_channel_decode", int),
}

# Read by other parts of the library, not by this module: accepted here so that setting them does
# not make the configuration fail ("EPX_NODE_ID": node label of the multi-node context).
# "EPX_MAX_TOKENS", "EPX_CUDA_GRAPH", "EPX_GEMM_CTA_PAIRS": read by the SGLang binding (per-rank
# token capacity, full decode graphs on/off, CTA pairs in the grouped GEMM).
_FOREIGN = ("EPX_NODE_ID", "EPX_MAX_TOKENS", "EPX_CUDA_GRAPH", "EPX_GEMM_CTA_PAIRS")

PRESETS = {
    # decode-heavy serving: small bounded batches, many retained per-layer workspaces
    "b200_decode": {"EPX_TRANSPORT": "nvlink", "EPX_DECODE_MAX_TOKENS": "256", "EPX_SLOTS": "2",
                    "EPX_WORKSPACE_POOL_BYTES": str(8 << 30), "EPX_TIMEOUT_SECONDS": "30"},
    # prefill-heavy: large slots, default workspace reserve
    "b200_prefill": {"EPX_TRANSPORT": "nvlink", "EPX_SLOTS": "2", "EPX_TIMEOUT_SECONDS": "60"},
    # the host-staged oracle path, for debugging a deployment without NVLink
    "host_oracle": {"EPX_TRANSPORT": "host_ce", "EPX_TIMEOUT_SECONDS": "120"},
}


def _parse(name, kind, text):
    try:
        if kind == "bool":
            if text.lower() in ("1", "true", "yes", "on"):
                return True
            if text.lower() in ("0", "false", "no", "off"):
                return False
            raise ValueError
        return kind(text)
    except ValueError:
        raise ValueError(f"{name}={text!r} is not a valid value") from None


def config_from_env(hidden_size, topk, max_tokens_per_rank, env=None, preset=None, **overrides):
    """Build a validated ``Config``: preset < environment < explicit overrides."""
    env = os.environ if env is None else env
    preset = env.get("EPX_PRESET", preset)
    values = {}
    if preset is not None:
        if preset not in PRESETS:
            raise ValueError(f"unknown preset {preset!r}; choose from {sorted(PRESETS)}")
        values.update(PRESETS[preset])
    unknown = [k for k in env if k.startswith("EPX_") and k not in _FIELDS and k not in _POLICY
               and k not in _FOREIGN and k != "EPX_PRESET"]
    if unknown:
        raise ValueError(f"unknown configuration variables: {sorted(unknown)}")
    values.update({k: v for k, v in env.items() if k in _FIELDS})
    kwargs = {}
    for name, text in values.items():
        field, kind = _FIELDS[name]
        kwargs[field] = _parse(name, kind, text)
    kwargs.update(overrides)
    return Config(hidden_size=hidden_size, topk=topk, max_tokens_per_rank=max_tokens_per_rank, **kwargs)


def channel_policy_from_env(env=None):
    """Keyword arguments for ``select_active_channels`` / ``EPDispatcher(channel_policy=...)``."""
    env = os.environ if env is None else env
    policy = {}
    for name, (key, kind) in _POLICY.items():
        if name in env:
            policy[key] = _parse(name, kind, env[name])
    if policy.get("tokens_per_channel_decode", 1) < 1:
        raise ValueError("EPX_DECODE_TOKENS_PER_CHANNEL must be positive")
    return policy
