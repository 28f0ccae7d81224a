// Grouped SwiGLU expert GEMM for sm_100a: tcgen05.mma with TMEM accumulators, operands
// staged in shared memory by TMA, one elected thread issuing the MMAs.
//
// The reference ships no expert GEMM: its adapter calls a framework's Triton kernel
// around count-aware helper kernels (ep_xpress/adapters/sglang_valid.py:13-255). This
// file is the hand-written replacement for that whole runner:
//
//   align      received (row, slot) pairs whose expert lives on this rank are grouped by
//              expert into 128-row tiles bounded by the DEVICE valid_count (the job of
//              sglang_valid.py:13-161);
//   gather     activation rows are permuted into that expert-sorted order;
//   GEMM 1     act = silu(x W1_e) * (x W3_e): gate and up columns of one output tile are
//              accumulated side by side in TMEM (128 x 256 FP32) and fused in the epilogue
//              (the framework needs a separate activation kernel,
//              adapters/sglang/sglang-v0.5.21.patch:281-330);
//   GEMM 2     y = (act W2_e) * routing weight, rounded to BF16 per (row, slot);
//   slot sum   partial[row] = bf16(sum over the row's local slots, in slot order, FP32) -
//              the definition of a rank's partial (sglang_valid.py:206-222).
//
// Kernel structure (both GEMMs): persistent CTAs of 192 threads. Warp 0 elects one thread
// that drives TMA loads into a 4-stage ring of 128B-swizzled K-major tiles; warp 1 elects
// one thread that issues tcgen05.mma (M 128, N 256, K 16) and commits stage releases and
// accumulator hand-offs to mbarriers; warps 2-5 are the epilogue, each owning the 32 TMEM
// lanes of its quadrant. Two accumulator buffers (2 x 256 TMEM columns) let the epilogue of
// one tile overlap the main loop of the next. Every wait is bounded and ends in an error
// flag, after which TMEM is still released.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "epx_device.cuh"
#include "moe_gemm.h"

namespace epx {
namespace {

constexpr int kTileM = 128;
constexpr int kTileN = 256;
constexpr int kTileK = 64;                 // 64 BF16 = one 128-byte swizzle row
constexpr int kGemmStages = 4;
constexpr int kABytes = kTileM * kTileK * 2;
constexpr int kBBytes = kTileN * kTileK * 2;
constexpr int kStageBytesGemm = kABytes + kBBytes;
constexpr int kGemmThreads = 192;
constexpr int kAccumColumns = 256;
constexpr unsigned long long kGemmWaitNs = 2000000000ull;   // bound of every pipeline wait: 2 s

// ---- PTX wrappers ----------------------------------------------------------------------
__device__ __forceinline__ bool elect_one() {
  unsigned pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_address(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
  return mbarrier_wait_bounded(bar, parity, kGemmWaitNs);
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_address(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_address(bar)) : "memory");
}
// Four rows of a row-major matrix (any four row indices) x one 64-column box, written to `dst`
// as four consecutive 128-byte rows; the tensor map has a box of {64, 1}. A row index at or
// beyond the matrix height reads zeros. No fan-out: the copy lands in this CTA only.
__device__ __forceinline__ void tma_gather4(void* dst, const CUtensorMap* map, int x, int r0, int r1, int r2, int r3,
                                            unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
      ::"r"(smem_address(dst)), "l"(map), "r"(x), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(smem_address(bar))
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(unsigned* smem_result, unsigned columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_address(smem_result)), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned address, unsigned columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc,
                                          unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on `bar` once every MMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_address(bar)) : "memory");
}
__device__ __forceinline__ void tmem_load_32(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 BF16) and
// 128-byte swizzled: 8-row groups are 1024 bytes apart (stride byte offset), the leading
// byte offset is unused for swizzled K-major layouts, descriptor version 1, layout type 2.
__device__ __forceinline__ unsigned long long smem_descriptor(const void* tile) {
  const unsigned long long address = smem_address(tile);
  return ((address & 0x3ffffull) >> 4) | (1ull << 16) | ((1024ull >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: D FP32, A/B BF16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ constexpr unsigned instruction_descriptor(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<unsigned>(n >> 3) << 17) |
         (static_cast<unsigned>(m >> 4) << 24);
}


// ---- the grouped GEMM kernel -------------------------------------------------------------------
struct GemmParams {
  const int* num_m_tiles;        // device: 128-row tiles in use (depends on routing)
  const int* tile_expert;        // device: [max tiles] local expert of each tile
  const float* row_scale;        // kMode 1: routing weight of every sorted row
  void* out;                     // bf16 [padded rows, out_columns]
  int* error_flag;               // set to 1 when a bounded wait gave up
  int k_steps;                   // K / 64
  int n_tiles;                   // output column tiles per row tile
  int out_columns;               // row pitch of `out` in elements
  int b_rows_per_expert;         // rows of the weight matrix that belong to one expert
  int up_row_offset;             // kMode 0: row distance between gate and up projections
  const int* gather_rows;        // null, or [padded rows]: source row of every sorted position (-1: padding);
                                 // the A operand is then gathered from the unsorted matrix behind map_a
  int gather_height;             // rows of that matrix; an index at or above it reads zeros
};

// Row indices of lane `lane`'s four rows of the 128-row block that starts at `first`.
__device__ __forceinline__ int4 gather_indices(const GemmParams& p, long long first, int lane) {
  int4 rows = *reinterpret_cast<const int4*>(p.gather_rows + first + 4 * lane);
  if (rows.x < 0) rows.x = p.gather_height;
  if (rows.y < 0) rows.y = p.gather_height;
  if (rows.z < 0) rows.z = p.gather_height;
  if (rows.w < 0) rows.w = p.gather_height;
  return rows;
}

// kMode 0: B tile = [128 gate rows; 128 up rows], epilogue silu(gate) * up -> 128 columns.
// kMode 1: B tile = 256 rows, epilogue acc * row_scale -> 256 columns.
template <int kMode>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p) {
  extern __shared__ __align__(1024) unsigned char gemm_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023) &
                                                         ~static_cast<uintptr_t>(1023));
  __shared__ unsigned long long full_bar[kGemmStages], empty_bar[kGemmStages];
  __shared__ unsigned long long acc_full[2], acc_empty[2];
  __shared__ unsigned tmem_base_slot;
  __shared__ volatile int failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kGemmStages; ++s) {
      mbarrier_init(full_bar + s, 1);
      mbarrier_init(empty_bar + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbarrier_init(acc_full + b, 1);
      mbarrier_init(acc_empty + b, 4);          // one arrival per epilogue warp
    }
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  if (warp == 1) tmem_alloc(&tmem_base_slot, 2 * kAccumColumns);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const unsigned tmem_base = tmem_base_slot;

  const int m_tiles = *p.num_m_tiles;
  const long long total_tiles = static_cast<long long>(m_tiles) * p.n_tiles;
  constexpr int kOutTile = kMode == 0 ? kTileN / 2 : kTileN;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (p.gather_rows != nullptr) {
      // Gathered A operand: the whole warp takes part, lane l fetches rows 4l..4l+3 of the tile
      // with ONE gather copy per k-step straight from the unsorted activation matrix.
      unsigned use = 0;
      bool go = true;
      for (long long tile = blockIdx.x; tile < total_tiles && go; tile += gridDim.x) {
        const int m_tile = static_cast<int>(tile / p.n_tiles), n_tile = static_cast<int>(tile % p.n_tiles);
        const int expert = p.tile_expert[m_tile];
        const int b_row = expert * p.b_rows_per_expert + n_tile * kOutTile;
        const int4 rows = gather_indices(p, static_cast<long long>(m_tile) * kTileM, lane);
        for (int k = 0; k < p.k_steps && go; ++k, ++use) {
          const int s = use % kGemmStages;
          unsigned char* a_dst = smem + static_cast<size_t>(s) * kStageBytesGemm;
          unsigned char* b_dst = a_dst + kABytes;
          int ok = 1;
          if (lane == 0) {
            ok = !failed && mbar_wait(empty_bar + s, ((use / kGemmStages) & 1u) ^ 1u) ? 1 : 0;
            if (ok) mbarrier_arrive_expect_tx(full_bar + s, kStageBytesGemm);
            else failed = 1;
          }
          go = __shfl_sync(0xffffffffu, ok, 0) != 0;
          if (!go) break;
          tma_gather4(a_dst + lane * 512, &map_a, k * kTileK, rows.x, rows.y, rows.z, rows.w, full_bar + s);
          if (lane == 0) {
            if (kMode == 0) {
              tma_load_2d(b_dst, &map_b, k * kTileK, b_row, full_bar + s);
              tma_load_2d(b_dst + kBBytes / 2, &map_b, k * kTileK, b_row + p.up_row_offset, full_bar + s);
            } else {
              tma_load_2d(b_dst, &map_b, k * kTileK, b_row, full_bar + s);
            }
          }
        }
      }
    } else if (elect_one()) {
      unsigned use = 0;
      for (long long tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x) {
        const int m_tile = static_cast<int>(tile / p.n_tiles), n_tile = static_cast<int>(tile % p.n_tiles);
        const int expert = p.tile_expert[m_tile];
        const int b_row = expert * p.b_rows_per_expert + n_tile * kOutTile;
        for (int k = 0; k < p.k_steps; ++k, ++use) {
          const int s = use % kGemmStages;
          if (!mbar_wait(empty_bar + s, ((use / kGemmStages) & 1u) ^ 1u)) { failed = 1; break; }
          unsigned char* a_dst = smem + static_cast<size_t>(s) * kStageBytesGemm;
          unsigned char* b_dst = a_dst + kABytes;
          mbarrier_arrive_expect_tx(full_bar + s, kStageBytesGemm);
          tma_load_2d(a_dst, &map_a, k * kTileK, m_tile * kTileM, full_bar + s);
          if (kMode == 0) {
            tma_load_2d(b_dst, &map_b, k * kTileK, b_row, full_bar + s);
            tma_load_2d(b_dst + kBBytes / 2, &map_b, k * kTileK, b_row + p.up_row_offset, full_bar + s);
          } else {
            tma_load_2d(b_dst, &map_b, k * kTileK, b_row, full_bar + s);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr unsigned idesc = instruction_descriptor(kTileM, kTileN);
      unsigned use = 0, local_tile = 0;
      for (long long tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x, ++local_tile) {
        const unsigned buffer = local_tile & 1u;
        if (!mbar_wait(acc_empty + buffer, ((local_tile >> 1) & 1u) ^ 1u)) { failed = 1; break; }
        tcgen05_fence_after();
        const unsigned tmem_d = tmem_base + buffer * kAccumColumns;
        for (int k = 0; k < p.k_steps; ++k, ++use) {
          const int s = use % kGemmStages;
          if (!mbar_wait(full_bar + s, (use / kGemmStages) & 1u)) { failed = 1; break; }
          tcgen05_fence_after();
          const unsigned char* a_tile = smem + static_cast<size_t>(s) * kStageBytesGemm;
          const unsigned long long a_desc = smem_descriptor(a_tile);
          const unsigned long long b_desc = smem_descriptor(a_tile + kABytes);
#pragma unroll
          for (int kk = 0; kk < kTileK / 16; ++kk)   // 16 BF16 = 32 bytes = 2 descriptor units per step
            umma_bf16(tmem_d, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (k | kk) != 0 ? 1u : 0u);
          umma_commit(empty_bar + s);                 // stage reusable when these MMAs retire
        }
        if (failed) break;
        umma_commit(acc_full + buffer);               // accumulator complete
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5, TMEM lane quadrant = warp % 4 ----------------
    const int quadrant = warp & 3;
    const int row_in_tile = quadrant * 32 + lane;
    unsigned local_tile = 0;
    for (long long tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local_tile) {
      const int m_tile = static_cast<int>(tile / p.n_tiles), n_tile = static_cast<int>(tile % p.n_tiles);
      const unsigned buffer = local_tile & 1u;
      const bool ok = mbar_wait(acc_full + buffer, (local_tile >> 1) & 1u);
      if (!__all_sync(0xffffffffu, ok)) { failed = 1; break; }
      tcgen05_fence_after();
      const unsigned taddr = tmem_base + buffer * kAccumColumns + (static_cast<unsigned>(quadrant * 32) << 16);
      const long long row = static_cast<long long>(m_tile) * kTileM + row_in_tile;
      __nv_bfloat16* out_row = reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.out_columns +
                               static_cast<long long>(n_tile) * kOutTile;
      const float scale = kMode == 1 ? p.row_scale[row] : 1.f;
#pragma unroll 1
      for (int chunk = 0; chunk < kOutTile / 32; ++chunk) {
        unsigned first[32];
        unsigned second[32];
        tmem_load_32(taddr + chunk * 32, first);
        if (kMode == 0) tmem_load_32(taddr + kTileN / 2 + chunk * 32, second);
        tmem_load_wait();
        unsigned packed[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float lo, hi;
          if (kMode == 0) {
            const float g0 = __uint_as_float(first[2 * i]), g1 = __uint_as_float(first[2 * i + 1]);
            lo = (g0 / (1.f + __expf(-g0))) * __uint_as_float(second[2 * i]);
            hi = (g1 / (1.f + __expf(-g1))) * __uint_as_float(second[2 * i + 1]);
          } else {
            lo = __uint_as_float(first[2 * i]) * scale;
            hi = __uint_as_float(first[2 * i + 1]) * scale;
          }
          packed[i] = pack_bf16x2(lo, hi);
        }
        uint4* dst = reinterpret_cast<uint4*>(out_row + chunk * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q)
          dst[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + buffer);
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 2 * kAccumColumns);
  }
  if (threadIdx.x == 0 && failed) atomicExch(p.error_flag, 1);
}


// ---- the same GEMM on CTA pairs (thread-block clusters of two, tcgen05 cta_group::2) ------------
// One 128 x 256 tile per SM needs 48 KB of operands per k-step; at full tensor rate that is
// more L2 bandwidth x latency than four stages of shared memory can keep in flight. A pair
// of CTAs computes a 256 x 256 tile instead: each CTA stages its own 128 rows of A and HALF
// of the B tile (32 KB per k-step, six stages), the leader CTA's elected thread issues
// tcgen05.mma.cta_group::2 which reads both CTAs' shared memory and writes each CTA's half
// of the accumulator into that CTA's own TMEM, and both CTAs run their own epilogue. Both
// producers complete their TMA loads on the LEADER's full barrier; the leader commits stage
// releases and accumulator hand-offs to both CTAs' barriers. No load fans out to more than
// one CTA: each CTA fetches exactly the bytes it keeps.
constexpr int kPairStages = 6;
constexpr int kPairBBytes = kBBytes / 2;
constexpr int kPairStageBytes = kABytes + kPairBBytes;
constexpr size_t kPairSmemBytes = static_cast<size_t>(kPairStages) * kPairStageBytes + 1024;

__device__ __forceinline__ unsigned cluster_ctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory object in CTA `rank` of this cluster.
__device__ __forceinline__ unsigned peer_smem_address(const void* local, unsigned rank) {
  unsigned out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_address(local)), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_address) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_address) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, unsigned bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_address(dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void tma_gather4_pair(void* dst, const CUtensorMap* map, int x, int r0, int r1, int r2, int r3,
                                                 unsigned bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes.cta_group::2 "
      "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
      ::"r"(smem_address(dst)), "l"(map), "r"(x), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(unsigned* smem_result, unsigned columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_address(smem_result)), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(unsigned address, unsigned columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc,
                                               unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(unsigned bar_cluster) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster)
               : "memory");
}

template <int kMode>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const GemmParams p) {
  extern __shared__ __align__(1024) unsigned char gemm_smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023) &
                                                         ~static_cast<uintptr_t>(1023));
  __shared__ unsigned long long full_bar[kPairStages], empty_bar[kPairStages];
  __shared__ unsigned long long acc_full[2], acc_empty[2];
  __shared__ unsigned tmem_base_slot;
  __shared__ volatile int failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = cluster_ctarank();           // 0 = leader
  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbarrier_init(full_bar + s, 1);                // leader's: one arrive.expect_tx + both CTAs' bytes
      mbarrier_init(empty_bar + s, 1);               // one commit from the leader per use
    }
    for (int b = 0; b < 2; ++b) {
      mbarrier_init(acc_full + b, 1);                // one commit from the leader per tile
      mbarrier_init(acc_empty + b, 8);               // leader's: four epilogue warps of each CTA
    }
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  if (warp == 1) tmem_alloc_pair(&tmem_base_slot, 2 * kAccumColumns);
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync();                                    // both CTAs' barriers exist before anyone signals
  tcgen05_fence_after();
  const unsigned tmem_base = tmem_base_slot;

  const int m_tiles = *p.num_m_tiles;                // 256-row tiles
  const long long total_tiles = static_cast<long long>(m_tiles) * p.n_tiles;
  const long long cluster_id = blockIdx.x / 2, clusters = gridDim.x / 2;
  constexpr int kOutTile = kMode == 0 ? kTileN / 2 : kTileN;
  constexpr int kPairM = 2 * kTileM;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (p.gather_rows != nullptr) {
      // Gathered A operand (see the single-CTA kernel): each CTA gathers its own 128 rows.
      unsigned use = 0;
      bool go = true;
      for (long long tile = cluster_id; tile < total_tiles && go; tile += clusters) {
        const int m_tile = static_cast<int>(tile / p.n_tiles), n_tile = static_cast<int>(tile % p.n_tiles);
        const int expert = p.tile_expert[m_tile];
        const int b_row = expert * p.b_rows_per_expert + n_tile * kOutTile +
                          (kMode == 0 ? static_cast<int>(rank) * p.up_row_offset : static_cast<int>(rank) * (kTileN / 2));
        const int4 rows = gather_indices(p, static_cast<long long>(m_tile) * kPairM + static_cast<long long>(rank) * kTileM, lane);
        for (int k = 0; k < p.k_steps && go; ++k, ++use) {
          const int s = use % kPairStages;
          unsigned char* a_dst = smem + static_cast<size_t>(s) * kPairStageBytes;
          const unsigned leader_full = peer_smem_address(full_bar + s, 0);
          int ok = 1;
          if (lane == 0) {
            ok = !failed && mbar_wait(empty_bar + s, ((use / kPairStages) & 1u) ^ 1u) ? 1 : 0;
            if (!ok) failed = 1;
            else if (rank == 0) mbarrier_arrive_expect_tx(full_bar + s, 2 * kPairStageBytes);
          }
          go = __shfl_sync(0xffffffffu, ok, 0) != 0;
          if (!go) break;
          tma_gather4_pair(a_dst + lane * 512, &map_a, k * kTileK, rows.x, rows.y, rows.z, rows.w, leader_full);
          if (lane == 0) tma_load_2d_pair(a_dst + kABytes, &map_b, k * kTileK, b_row, leader_full);
        }
      }
    } else if (elect_one()) {
      unsigned use = 0;
      for (long long tile = cluster_id; tile < total_tiles && !failed; tile += clusters) {
        const int m_tile = static_cast<int>(tile / p.n_tiles), n_tile = static_cast<int>(tile % p.n_tiles);
        const int expert = p.tile_expert[m_tile];
        // Mode 0: the leader keeps the gate rows, its peer the up rows. Mode 1: halves of the tile.
        const int b_row = expert * p.b_rows_per_expert + n_tile * kOutTile +
                          (kMode == 0 ? static_cast<int>(rank) * p.up_row_offset : static_cast<int>(rank) * (kTileN / 2));
        for (int k = 0; k < p.k_steps; ++k, ++use) {
          const int s = use % kPairStages;
          if (!mbar_wait(empty_bar + s, ((use / kPairStages) & 1u) ^ 1u)) { failed = 1; break; }
          unsigned char* a_dst = smem + static_cast<size_t>(s) * kPairStageBytes;
          const unsigned leader_full = peer_smem_address(full_bar + s, 0);
          if (rank == 0) mbarrier_arrive_expect_tx(full_bar + s, 2 * kPairStageBytes);
          tma_load_2d_pair(a_dst, &map_a, k * kTileK, m_tile * kPairM + static_cast<int>(rank) * kTileM, leader_full);
          tma_load_2d_pair(a_dst + kABytes, &map_b, k * kTileK, b_row, leader_full);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader only) ----------------
    if (rank == 0 && elect_one()) {
      constexpr unsigned idesc = instruction_descriptor(kPairM, kTileN);
      unsigned use = 0, local_tile = 0;
      for (long long tile = cluster_id; tile < total_tiles && !failed; tile += clusters, ++local_tile) {
        const unsigned buffer = local_tile & 1u;
        if (!mbar_wait(acc_empty + buffer, ((local_tile >> 1) & 1u) ^ 1u)) { failed = 1; break; }
        tcgen05_fence_after();
        const unsigned tmem_d = tmem_base + buffer * kAccumColumns;
        for (int k = 0; k < p.k_steps; ++k, ++use) {
          const int s = use % kPairStages;
          if (!mbar_wait(full_bar + s, (use / kPairStages) & 1u)) { failed = 1; break; }
          tcgen05_fence_after();
          const unsigned char* a_tile = smem + static_cast<size_t>(s) * kPairStageBytes;
          const unsigned long long a_desc = smem_descriptor(a_tile);
          const unsigned long long b_desc = smem_descriptor(a_tile + kABytes);
#pragma unroll
          for (int kk = 0; kk < kTileK / 16; ++kk)
            umma_bf16_pair(tmem_d, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (k | kk) != 0 ? 1u : 0u);
          umma_commit_pair(peer_smem_address(empty_bar + s, 0));     // both CTAs may refill the stage
          umma_commit_pair(peer_smem_address(empty_bar + s, 1));
        }
        if (failed) break;
        umma_commit_pair(peer_smem_address(acc_full + buffer, 0));   // both epilogues may read
        umma_commit_pair(peer_smem_address(acc_full + buffer, 1));
      }
    }
  } else {
    // ---------------- epilogue (both CTAs, own 128 rows) ----------------
    const int quadrant = warp & 3;
    const int row_in_tile = static_cast<int>(rank) * kTileM + quadrant * 32 + lane;
    unsigned local_tile = 0;
    for (long long tile = cluster_id; tile < total_tiles; tile += clusters, ++local_tile) {
      const int m_tile = static_cast<int>(tile / p.n_tiles), n_tile = static_cast<int>(tile % p.n_tiles);
      const unsigned buffer = local_tile & 1u;
      const bool ok = mbar_wait(acc_full + buffer, (local_tile >> 1) & 1u);
      if (!__all_sync(0xffffffffu, ok)) { failed = 1; break; }
      tcgen05_fence_after();
      const unsigned taddr = tmem_base + buffer * kAccumColumns + (static_cast<unsigned>(quadrant * 32) << 16);
      const long long row = static_cast<long long>(m_tile) * kPairM + row_in_tile;
      __nv_bfloat16* out_row = reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.out_columns +
                               static_cast<long long>(n_tile) * kOutTile;
      const float scale = kMode == 1 ? p.row_scale[row] : 1.f;
#pragma unroll 1
      for (int chunk = 0; chunk < kOutTile / 32; ++chunk) {
        unsigned first[32];
        unsigned second[32];
        tmem_load_32(taddr + chunk * 32, first);
        if (kMode == 0) tmem_load_32(taddr + kTileN / 2 + chunk * 32, second);
        tmem_load_wait();
        unsigned packed[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float lo, hi;
          if (kMode == 0) {
            const float g0 = __uint_as_float(first[2 * i]), g1 = __uint_as_float(first[2 * i + 1]);
            lo = (g0 / (1.f + __expf(-g0))) * __uint_as_float(second[2 * i]);
            hi = (g1 / (1.f + __expf(-g1))) * __uint_as_float(second[2 * i + 1]);
          } else {
            lo = __uint_as_float(first[2 * i]) * scale;
            hi = __uint_as_float(first[2 * i + 1]) * scale;
          }
          packed[i] = pack_bf16x2(lo, hi);
        }
        uint4* dst = reinterpret_cast<uint4*>(out_row + chunk * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q)
          dst[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(peer_smem_address(acc_empty + buffer, 0));   // the leader's barrier
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync();                                    // the peer is done with this CTA's barriers and TMEM
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, 2 * kAccumColumns);
  }
  if (threadIdx.x == 0 && failed) atomicExch(p.error_flag, 1);
}

// ---- align / gather / slot-sum helper kernels ---------------------------------------------------
constexpr int kAlignThreads = 1024;
constexpr int kMaxLocalExperts = 1024;

__global__ void __launch_bounds__(256) moe_fill_kernel(int* sorted_row, float* sorted_scale, long long sorted_rows,
                                                       int* entry_pos, long long entries) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long me = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (long long i = me; i < sorted_rows; i += stride) { sorted_row[i] = -1; sorted_scale[i] = 0.f; }
  for (long long i = me; i < entries; i += stride) entry_pos[i] = -1;
}

// One CTA: histogram per local expert, tile-padded prefix, scatter. Bounded by the device
// valid_count, never by a host-side count.
__global__ void __launch_bounds__(kAlignThreads) moe_align_kernel(const long long* __restrict__ local_ids,
                                                                  const float* __restrict__ weights,
                                                                  const int* __restrict__ valid_count, int rows,
                                                                  int topk, int experts, long long max_sorted_rows,
                                                                  int max_tiles, int tile, int* sorted_row, float* sorted_scale,
                                                                  int* entry_pos, int* tile_expert, int* counters,
                                                                  int* error_flag) {
  __shared__ int s_count[kMaxLocalExperts];
  __shared__ int s_offset[kMaxLocalExperts];
  const int valid = min(*valid_count, rows);
  const long long pairs = static_cast<long long>(valid) * topk;
  for (int e = threadIdx.x; e < experts; e += kAlignThreads) s_count[e] = 0;
  __syncthreads();
  for (long long i = threadIdx.x; i < pairs; i += kAlignThreads) {
    const long long id = local_ids[i];
    if (id >= 0 && id < experts) atomicAdd(&s_count[id], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int offset = 0, tiles = 0;
    for (int e = 0; e < experts; ++e) {
      const int padded = (s_count[e] + tile - 1) / tile * tile;
      s_offset[e] = offset;
      for (int t = 0; t < padded / tile && tiles < max_tiles; ++t) tile_expert[tiles++] = e;
      offset += padded;
    }
    if (offset > max_sorted_rows) {           // the caller's bound on local pairs was too small
      atomicExch(error_flag, 2);
      offset = static_cast<int>(max_sorted_rows);
    }
    counters[0] = tiles < offset / tile ? tiles : offset / tile;
    counters[1] = offset;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += kAlignThreads) s_count[e] = 0;
  __syncthreads();
  for (long long i = threadIdx.x; i < pairs; i += kAlignThreads) {
    const long long id = local_ids[i];
    if (id < 0 || id >= experts) continue;
    const long long pos = s_offset[id] + atomicAdd(&s_count[id], 1);
    if (pos >= max_sorted_rows) continue;
    sorted_row[pos] = static_cast<int>(i / topk);
    sorted_scale[pos] = weights[i];
    entry_pos[i] = static_cast<int>(pos);
  }
}

__global__ void __launch_bounds__(256) moe_gather_kernel(const uint4* __restrict__ hidden, const int* __restrict__ sorted_row,
                                                         const int* __restrict__ counters, uint4* __restrict__ sorted_x,
                                                         long long max_sorted_rows, int vecs_per_row) {
  const long long used = min(static_cast<long long>(counters[1]), max_sorted_rows);
  const int lane = threadIdx.x & 31;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x / 32);
  for (long long pos = static_cast<long long>(blockIdx.x) * (blockDim.x / 32) + (threadIdx.x >> 5); pos < used;
       pos += warps) {
    const int row = sorted_row[pos];
    uint4* dst = sorted_x + pos * vecs_per_row;
    const uint4* src = hidden + static_cast<long long>(row < 0 ? 0 : row) * vecs_per_row;
    for (int base = lane; base < vecs_per_row; base += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (base + u * 32 < vecs_per_row) v[u] = row < 0 ? make_uint4(0, 0, 0, 0) : src[base + u * 32];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (base + u * 32 < vecs_per_row) dst[base + u * 32] = v[u];
    }
  }
}

__global__ void __launch_bounds__(256) moe_slot_sum_kernel(const uint4* __restrict__ y, const int* __restrict__ entry_pos,
                                                           const int* __restrict__ valid_count, uint4* __restrict__ partial,
                                                           int rows, int topk, int vecs_per_row) {
  const int valid = min(*valid_count, rows);
  const int lane = threadIdx.x & 31;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x / 32);
  for (long long row = static_cast<long long>(blockIdx.x) * (blockDim.x / 32) + (threadIdx.x >> 5); row < valid;
       row += warps) {
    // Lane k holds the sorted position of slot k (fetched once per row, not once per chunk).
    const int slots = min(topk, 32);
    const int my_pos = lane < slots ? entry_pos[row * topk + lane] : -1;
    for (int start = 0; start < vecs_per_row; start += 64) {          // warp-uniform; two chunks per lane in flight
      const int base = start + lane;
      float acc[2][8];
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[u][i] = 0.f;
      for (int k = 0; k < topk; ++k) {
        const int pos = k < 32 ? __shfl_sync(0xffffffffu, my_pos, k) : entry_pos[row * topk + k];
        if (pos < 0) continue;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int at = base + u * 32;
          if (at < vecs_per_row) {
            const uint4 v = y[static_cast<long long>(pos) * vecs_per_row + at];
            const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              acc[u][2 * i] = __fadd_rn(acc[u][2 * i], __uint_as_float(w[i] << 16));
              acc[u][2 * i + 1] = __fadd_rn(acc[u][2 * i + 1], __uint_as_float(w[i] & 0xffff0000u));
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int at = base + u * 32;
        if (at < vecs_per_row) {
          unsigned out[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            out[i] = pack_bf16x2(acc[u][2 * i], acc[u][2 * i + 1]);
          partial[row * vecs_per_row + at] = make_uint4(out[0], out[1], out[2], out[3]);
        }
      }
    }
  }
}

// ---- tensor maps ----------------------------------------------------------------------------------
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled fn = [] {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
      entry = nullptr;
    return reinterpret_cast<EncodeTiled>(entry);
  }();
  return fn;
}

// Row-major BF16 matrix [rows, columns]; box = box_rows x 64 columns, 128-byte swizzle.
cudaError_t make_map(CUtensorMap* map, const void* base, long long rows, long long columns, int box_rows) {
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return cudaErrorNotSupported;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(columns), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(columns) * 2};
  const cuuint32_t box[2] = {kTileK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t element_strides[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                            element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// Same matrix addressed one row at a time (box 1 x 64 columns): the form gather copies need.
cudaError_t make_gather_map(CUtensorMap* map, const void* base, long long rows, long long columns) {
  return make_map(map, base, rows, columns, 1);
}

constexpr size_t kGemmSmemBytes = static_cast<size_t>(kGemmStages) * kStageBytesGemm + 1024;

template <int kMode>
cudaError_t launch_gemm_pair(const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmParams& params, int sms,
                             cudaStream_t stream) {
  cudaError_t err = cudaFuncSetAttribute(grouped_gemm_pair_kernel<kMode>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kPairSmemBytes));
  if (err != cudaSuccess) return err;
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(sms / 2 * 2, 1, 1);
  config.blockDim = dim3(kGemmThreads, 1, 1);
  config.dynamicSmemBytes = kPairSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = 2;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, grouped_gemm_pair_kernel<kMode>, map_a, map_b, params);
}

template <int kMode>
cudaError_t launch_gemm(const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmParams& params, int sms,
                        cudaStream_t stream) {
  cudaError_t err = cudaFuncSetAttribute(grouped_gemm_kernel<kMode>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kGemmSmemBytes));
  if (err != cudaSuccess) return err;
  grouped_gemm_kernel<kMode><<<sms, kGemmThreads, kGemmSmemBytes, stream>>>(map_a, map_b, params);
  return cudaGetLastError();
}

}  // namespace

MoeSizes moe_sizes(long long rows, int topk, int experts, int tile_rows) {
  const long long per_row = topk < experts ? topk : experts;
  const long long entries = rows * per_row;
  MoeSizes sizes;
  sizes.max_tiles = static_cast<int>((entries + tile_rows - 1) / tile_rows + experts);
  sizes.max_sorted_rows = static_cast<long long>(sizes.max_tiles) * tile_rows;
  return sizes;
}

cudaError_t launch_moe_align(const long long* local_ids, const float* weights, const int* valid_count, int rows,
                             int topk, int experts, long long max_sorted_rows, int max_tiles, int* sorted_row,
                             float* sorted_scale, int* entry_pos, int* tile_expert, int* counters,
                             int* error_flag, int tile_rows, cudaStream_t stream) {
  if (experts > kMaxLocalExperts || (tile_rows != kTileM && tile_rows != 2 * kTileM)) return cudaErrorInvalidValue;
  moe_fill_kernel<<<296, 256, 0, stream>>>(sorted_row, sorted_scale, max_sorted_rows, entry_pos,
                                           static_cast<long long>(rows) * topk);
  moe_align_kernel<<<1, kAlignThreads, 0, stream>>>(local_ids, weights, valid_count, rows, topk, experts,
                                                    max_sorted_rows, max_tiles, tile_rows, sorted_row, sorted_scale,
                                                    entry_pos, tile_expert, counters, error_flag);
  return cudaGetLastError();
}

cudaError_t launch_moe_gather(const void* hidden, const int* sorted_row, const int* counters, void* sorted_x,
                              long long max_sorted_rows, int hidden_size, cudaStream_t stream) {
  if (hidden_size % 8) return cudaErrorInvalidValue;
  moe_gather_kernel<<<148 * 8, 256, 0, stream>>>(static_cast<const uint4*>(hidden), sorted_row, counters,
                                                 static_cast<uint4*>(sorted_x), max_sorted_rows, hidden_size / 8);
  return cudaGetLastError();
}

cudaError_t launch_moe_gemm_gate_up(const void* sorted_x, const void* w13, void* act, const int* counters,
                                    const int* tile_expert, int* error_flag, long long max_sorted_rows,
                                    int experts, int hidden_size, int inter_size, int sms, bool pair,
                                    cudaStream_t stream, const int* gather_rows, long long gather_height) {
  if (hidden_size % kTileK || inter_size % kMoeGateUpTile) return cudaErrorInvalidValue;
  if (gather_rows != nullptr && (gather_height <= 0 || gather_height >= (1ll << 31) ||
                                 reinterpret_cast<uintptr_t>(gather_rows) % 16 != 0))
    return cudaErrorInvalidValue;
  CUtensorMap map_a, map_b;
  // With `gather_rows`, `sorted_x` is the UNSORTED activation matrix [gather_height, hidden].
  cudaError_t err = gather_rows != nullptr ? make_gather_map(&map_a, sorted_x, gather_height, hidden_size)
                                           : make_map(&map_a, sorted_x, max_sorted_rows, hidden_size, kTileM);
  if (err != cudaSuccess) return err;
  err = make_map(&map_b, w13, static_cast<long long>(experts) * 2 * inter_size, hidden_size, kTileN / 2);
  if (err != cudaSuccess) return err;
  GemmParams params{};
  params.num_m_tiles = counters;
  params.tile_expert = tile_expert;
  params.out = act;
  params.error_flag = error_flag;
  params.k_steps = hidden_size / kTileK;
  params.n_tiles = inter_size / kMoeGateUpTile;
  params.out_columns = inter_size;
  params.b_rows_per_expert = 2 * inter_size;
  params.up_row_offset = inter_size;
  params.gather_rows = gather_rows;
  params.gather_height = static_cast<int>(gather_height);
  return pair ? launch_gemm_pair<0>(map_a, map_b, params, sms, stream)
              : launch_gemm<0>(map_a, map_b, params, sms, stream);
}

cudaError_t launch_moe_gemm_down(const void* act, const void* w2, void* y, const float* sorted_scale,
                                 const int* counters, const int* tile_expert, int* error_flag,
                                 long long max_sorted_rows, int experts, int hidden_size, int inter_size, int sms,
                                 bool pair, cudaStream_t stream) {
  if (inter_size % kTileK || hidden_size % kMoeDownTile) return cudaErrorInvalidValue;
  CUtensorMap map_a, map_b;
  cudaError_t err = make_map(&map_a, act, max_sorted_rows, inter_size, kTileM);
  if (err != cudaSuccess) return err;
  err = make_map(&map_b, w2, static_cast<long long>(experts) * hidden_size, inter_size, pair ? kTileN / 2 : kTileN);
  if (err != cudaSuccess) return err;
  GemmParams params{};
  params.num_m_tiles = counters;
  params.tile_expert = tile_expert;
  params.row_scale = sorted_scale;
  params.out = y;
  params.error_flag = error_flag;
  params.k_steps = inter_size / kTileK;
  params.n_tiles = hidden_size / kMoeDownTile;
  params.out_columns = hidden_size;
  params.b_rows_per_expert = hidden_size;
  params.up_row_offset = 0;
  return pair ? launch_gemm_pair<1>(map_a, map_b, params, sms, stream)
              : launch_gemm<1>(map_a, map_b, params, sms, stream);
}

cudaError_t launch_moe_slot_sum(const void* y, const int* entry_pos, const int* valid_count, void* partial,
                                int rows, int topk, int hidden_size, cudaStream_t stream) {
  if (hidden_size % 8) return cudaErrorInvalidValue;
  if (rows <= 0) return cudaSuccess;
  const int ctas = rows < 148 * 8 * 8 ? (rows + 7) / 8 : 148 * 8;
  moe_slot_sum_kernel<<<ctas, 256, 0, stream>>>(static_cast<const uint4*>(y), entry_pos, valid_count,
                                                static_cast<uint4*>(partial), rows, topk, hidden_size / 8);
  return cudaGetLastError();
}

}  // namespace epx
