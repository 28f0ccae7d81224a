#!/usr/bin/env bash
# Eight B200s of one node, BF16, eager prefill and eager decode.
# usage: MODEL_PATH=/path/to/bf16/moe/checkpoint adapters/sglang/presets/nvlink_bf16_ep8.sh [more server flags]
set -euo pipefail
: "${MODEL_PATH:?set MODEL_PATH to a BF16 MoE checkpoint}"

export EPX_PRESET="${EPX_PRESET:-b200_prefill}"
export EPX_MAX_TOKENS="${EPX_MAX_TOKENS:-16384}"          # scheduled tokens per rank and forward, upper bound
export EPX_DECODE_MAX_TOKENS="${EPX_DECODE_MAX_TOKENS:-256}"
export EPX_CUDA_GRAPH="${EPX_CUDA_GRAPH:-0}"

exec python -m sglang.launch_server \
  --model-path "$MODEL_PATH" \
  --dtype bfloat16 \
  --tp-size 8 --ep-size 8 --dp-size 8 --enable-dp-attention \
  --moe-a2a-backend ep_xpress_b200 --moe-runner-backend triton \
  --cuda-graph-backend-decode disabled \
  --cuda-graph-backend-prefill disabled \
  "$@"
