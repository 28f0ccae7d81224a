#!/usr/bin/env bash
# Latency-oriented decode: graphs as in nvlink_bf16_ep8_graph.sh, small per-rank batches, one
# channel per four tokens so that a handful of tokens still spreads over several SMs.
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"

export EPX_DECODE_MAX_TOKENS="${EPX_DECODE_MAX_TOKENS:-64}"
export EPX_DECODE_TOKENS_PER_CHANNEL="${EPX_DECODE_TOKENS_PER_CHANNEL:-4}"
export EPX_MAX_TOKENS="${EPX_MAX_TOKENS:-8192}"

exec "$here/nvlink_bf16_ep8_graph.sh" "$@"
