#!/usr/bin/env bash
# As nvlink_bf16_ep8.sh, with the whole decode forward in CUDA graphs (prefill stays eager).
# Every graph bucket is warmed eagerly by SGLang before capture; that is when the per-layer
# workspaces and the expert runner's planes are allocated.
set -euo pipefail
: "${MODEL_PATH:?set MODEL_PATH to a BF16 MoE checkpoint}"

export EPX_PRESET="${EPX_PRESET:-b200_decode}"
export EPX_MAX_TOKENS="${EPX_MAX_TOKENS:-16384}"
export EPX_CUDA_GRAPH=1

exec python -m sglang.launch_server \
  --model-path "$MODEL_PATH" \
  --dtype bfloat16 \
  --tp-size 8 --ep-size 8 --dp-size 8 --enable-dp-attention \
  --moe-a2a-backend ep_xpress_b200 --moe-runner-backend triton \
  --cuda-graph-backend-decode full \
  --cuda-graph-backend-prefill disabled \
  "$@"
