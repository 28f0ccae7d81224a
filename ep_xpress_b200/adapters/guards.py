"""Deployment guards and launch-width policy (no framework import, no CUDA).

Same rules as the reference adapter (ep_xpress/adapters/sglang_config.py:6-116): the EP
group is the attention-DP group is the TP group, MoE tensor/data parallelism and pipeline
parallelism are off, experts sit in equal contiguous blocks, the receive capacity comes
from scheduler-known token counts, and the launch width follows the batch size.
"""

from __future__ import annotations


def validate_server_args(*, tp_size, dp_size, ep_size, pp_size=1, moe_tp_size=1, moe_dp_size=1,
                         enable_dp_attention=True):
    """Raise ValueError unless the parallel layout is one this library serves."""
    if pp_size != 1:
        raise ValueError("pipeline parallelism is not supported with the EP dispatcher (pp_size must be 1)")
    if not enable_dp_attention:
        raise ValueError("attention data parallelism is required: every rank owns its own tokens")
    if not (tp_size == dp_size == ep_size):
        raise ValueError("attention DP size, TP size and EP size must be equal")
    if moe_tp_size != 1 or moe_dp_size != 1:
        raise ValueError("MoE tensor and data parallelism must be 1: experts are sharded by EP only")
    if not 1 <= ep_size <= 63:
        raise ValueError("the EP group must have between 1 and 63 ranks")


def validate_runner_config(*, reduce_results, apply_router_weight_on_input=False, activation="silu"):
    """The expert runner must hand back already-weighted, not-yet-reduced partial rows."""
    if reduce_results:
        raise ValueError("reduce_results must be False: combine performs the cross-rank reduction")
    if apply_router_weight_on_input:
        raise ValueError("router weights are applied once, on the expert outputs")
    if activation != "silu":
        raise ValueError("the grouped expert runner implements SwiGLU (silu) only")


def contiguous_expert_map(num_experts, ep_size):
    if num_experts <= 0 or ep_size <= 0 or num_experts % ep_size:
        raise ValueError("experts must divide evenly into contiguous blocks per rank")
    per_rank = num_experts // ep_size
    return [expert // per_rank for expert in range(num_experts)]


def receive_capacity_from_scheduler(token_counts, max_tokens_per_rank):
    """CPU-known bound of received rows: the sum of every rank's scheduled tokens."""
    counts = [int(c) for c in token_counts]
    if not counts or any(c < 0 or c > max_tokens_per_rank for c in counts):
        raise ValueError("scheduler token counts must be within [0, max_tokens_per_rank] for every rank")
    return sum(counts)


def select_active_channels(tokens, effective_channels, *, is_decode, tokens_per_channel_decode=8, adaptive=True,
                           prefill_override=0, decode_override=0):
    """Channels (= share of the CTA budget) for one operation.

    A phase override asks for a fixed count and is clamped to what was allocated; with
    ``adaptive=False`` every operation uses all channels; otherwise prefill takes one channel
    per token and decode one per ``tokens_per_channel_decode`` tokens, up to all channels
    (the policy of the reference's adapter, ep_xpress/adapters/sglang_config.py:88-116). Each
    rank launches its own kernels and only synchronises its own CTAs, so ranks may arrive at
    different widths; pass the group's global token count when the same width is wanted
    everywhere.
    """
    if effective_channels < 1:
        raise ValueError("effective_channels must be positive")
    for name, value in (("prefill_override", prefill_override), ("decode_override", decode_override)):
        if isinstance(value, bool) or not isinstance(value, int) or value < 0:
            raise ValueError(f"{name} must be a non-negative integer")
    override = decode_override if is_decode else prefill_override
    if override:
        return min(effective_channels, override)
    if not adaptive:
        return effective_channels
    if tokens <= 0:
        return 1
    wanted = -(-tokens // tokens_per_channel_decode) if is_decode else tokens
    return max(1, min(effective_channels, wanted))


def validate_expert_runner(*, activation="silu", is_gated=True, gemm1_alpha=None, gemm1_clamp_limit=None,
                           swiglu_limit=None):
    """Static scope of the count-aware BF16 expert runner (``ops.GroupedSwiGLU``): gated SiLU
    without activation modifiers, checked once per model
    (ep_xpress/adapters/sglang_config.py:76-85)."""
    if activation != "silu" or not is_gated:
        raise ValueError("the grouped expert runner requires gated SiLU")
    if any(value is not None for value in (gemm1_alpha, gemm1_clamp_limit, swiglu_limit)):
        raise ValueError("the grouped expert runner does not support activation modifiers")


_UNSUPPORTED_SERVER_FEATURES = (
    "enable_eplb", "enable_waterfill", "enable_lora", "enable_two_batch_overlap", "enable_single_batch_overlap",
    "enable_fused_moe_sum_all_reduce", "enable_torch_compile", "speculative_algorithm", "ep_num_redundant_experts",
    "ep_join_mode", "elastic_ep_backend", "enable_memory_saver", "enable_pdmux",
)


def validate_serving_args(args, model_config=None):
    """The same layout rules for a serving framework's resolved argument OBJECT (attribute access,
    missing attributes take the framework's defaults), plus the features that would bypass or
    re-order the dispatcher. Scope of the reference's guard (ep_xpress/adapters/sglang_config.py:6-45)
    minus its model allow-list: any BF16 MoE with evenly split, unshared experts is served.
    """
    tp = getattr(args, "tp_size", 1)
    if getattr(args, "nnodes", 1) != 1:
        raise ValueError("the NVLink transport spans the GPUs of one node (nnodes must be 1)")
    validate_server_args(tp_size=tp, dp_size=getattr(args, "dp_size", 1), ep_size=getattr(args, "ep_size", tp),
                         pp_size=getattr(args, "pp_size", 1), moe_tp_size=getattr(args, "moe_tp_size", 1),
                         moe_dp_size=getattr(args, "moe_dp_size", 1),
                         enable_dp_attention=bool(getattr(args, "enable_dp_attention", False)))
    if getattr(args, "dwdp_size", 1) != 1:
        raise ValueError("dense-weight data parallelism is not supported with the EP dispatcher")
    if getattr(args, "dtype", None) not in ("bfloat16", "bf16"):
        raise ValueError("activations and expert weights must be BF16: pass the dtype explicitly")
    if getattr(args, "quantization", None) or getattr(model_config, "quantization_config", None):
        raise ValueError("quantised experts are not supported: the expert runner is BF16")
    for name in _UNSUPPORTED_SERVER_FEATURES:
        if getattr(args, name, None):
            raise ValueError(f"{name} is not supported with the EP dispatcher")
    if getattr(model_config, "n_shared_experts", 0) or getattr(model_config, "num_shared_experts", 0):
        raise ValueError("shared experts are not supported: every expert is routed")


def validate_moe_layer(config, *, world_size, bf16):
    """Per-layer facts of a framework's MoE runner configuration object: BF16, no fused shared
    experts, weighted output that is combined by the dispatcher, an even contiguous expert split
    (ep_xpress/adapters/sglang_config.py:48-58)."""
    if getattr(config, "params_dtype", bf16) != bf16:
        raise ValueError("the EP dispatcher needs BF16 activations and expert weights")
    if getattr(config, "num_fused_shared_experts", 0):
        raise ValueError("fused shared experts are not supported")
    validate_runner_config(reduce_results=False,
                           apply_router_weight_on_input=bool(getattr(config, "apply_router_weight_on_input", False)),
                           activation=getattr(config, "activation", "silu"))
    if getattr(config, "no_combine", False):
        raise ValueError("the expert runner must return combined-per-row output (no_combine is not supported)")
    if config.num_experts != world_size * config.num_local_experts:
        raise ValueError("experts must divide evenly into contiguous blocks per rank")
    if getattr(config, "use_tp_all_gather_activation", False):
        raise ValueError("TP activation all-gather cannot be combined with the EP dispatcher")
    validate_expert_runner(activation=getattr(config, "activation", "silu"), is_gated=getattr(config, "is_gated", True),
                           gemm1_alpha=getattr(config, "gemm1_alpha", None),
                           gemm1_clamp_limit=getattr(config, "gemm1_clamp_limit", None),
                           swiglu_limit=getattr(config, "swiglu_limit", None))
