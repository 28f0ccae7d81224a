// Host API of the grouped SwiGLU expert runner (plain C++, no torch types).
//
// The stages replace what the reference borrows from its serving framework and patches for a
// device-resident row count: route alignment (ep_xpress/adapters/sglang_valid.py:13-161), the
// grouped GEMMs with SiLU-and-mul in between (sglang_valid.py:233-255 and the act_and_mul patch,
// ep_xpress/adapters/sglang/sglang-v0.5.21.patch:281-330) and the slot-order FP32 sum with one
// BF16 rounding (sglang_valid.py:206-222).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace epx {

constexpr int kMoeTileRows = 128;     // rows of one expert-sorted tile
constexpr int kMoeGateUpTile = 128;   // intermediate columns produced by one GEMM-1 tile
constexpr int kMoeDownTile = 256;     // hidden columns produced by one GEMM-2 tile

struct MoeSizes {
  long long max_sorted_rows;   // upper bound of expert-sorted rows incl. tile padding
  int max_tiles;               // upper bound of 128-row tiles
};

// CPU-known bounds for `rows` received rows, `topk` slots per row and `experts` local experts.
// `tile_rows` is 128, or 256 when the GEMMs run on CTA pairs.
MoeSizes moe_sizes(long long rows, int topk, int experts, int tile_rows = kMoeTileRows);

// Groups the (row, slot) pairs of this rank's experts by expert into 128-row tiles.
//   sorted_row   int32 [max_sorted_rows]  source row of every sorted position, -1 = padding
//   sorted_scale f32   [max_sorted_rows]  routing weight of the pair, 0 for padding
//   entry_pos    int32 [rows * topk]      sorted position of the pair, -1 when not local
//   tile_expert  int32 [max_tiles]        local expert of every tile
//   counters     int32 [2]                {tiles in use, sorted rows in use}
//   error_flag   int32 [1]                set to 2 when max_sorted_rows was too small (pairs are dropped)
cudaError_t launch_moe_align(const long long* local_ids, const float* weights, const int* valid_count, int rows,
                             int topk, int experts, long long max_sorted_rows, int max_tiles, int* sorted_row,
                             float* sorted_scale, int* entry_pos, int* tile_expert, int* counters,
                             int* error_flag, int tile_rows, cudaStream_t stream);

// sorted_x[pos] = hidden[sorted_row[pos]] (zero rows for padding) for the tiles in use.
cudaError_t launch_moe_gather(const void* hidden, const int* sorted_row, const int* counters, void* sorted_x,
                              long long max_sorted_rows, int hidden_size, cudaStream_t stream);

// GEMM 1: act[pos, :] = silu(x W1_e) * (x W3_e).  w13 is [experts, 2 * inter, hidden] (gate rows
// first, then up rows), K-major. GEMM 2: y[pos, :] = (act W2_e) * sorted_scale[pos], w2 is
// [experts, hidden, inter]. Shapes: hidden % 256 == 0, inter % 128 == 0. `pair` runs the GEMM on
// clusters of two CTAs (tcgen05 cta_group::2, 256-row tiles: align with tile_rows = 256).
// With `gather_rows` (= the align step's sorted_row, 16-byte aligned), `sorted_x` is the UNSORTED
// activation matrix [gather_height, hidden]: the kernel's TMA producer gathers the rows of every
// tile itself (four rows per copy) and no gather launch or sorted copy of the activations is needed.
cudaError_t launch_moe_gemm_gate_up(const void* sorted_x, const void* w13, void* act, const int* counters,
                                    const int* tile_expert, int* error_flag, long long max_sorted_rows,
                                    int experts, int hidden_size, int inter_size, int sms, bool pair,
                                    cudaStream_t stream, const int* gather_rows = nullptr,
                                    long long gather_height = 0);
cudaError_t launch_moe_gemm_down(const void* act, const void* w2, void* y, const float* sorted_scale,
                                 const int* counters, const int* tile_expert, int* error_flag,
                                 long long max_sorted_rows, int experts, int hidden_size, int inter_size, int sms,
                                 bool pair, cudaStream_t stream);

// partial[row] = bf16(sum over slots, in slot order, of float(y[entry_pos[row, slot]])) for rows
// below *valid_count.
cudaError_t launch_moe_slot_sum(const void* y, const int* entry_pos, const int* valid_count, void* partial,
                                int rows, int topk, int hidden_size, cudaStream_t stream);

}  // namespace epx
