// Small helper kernels around the transport: the synthetic "identity times
// routing weight" expert used for validation and for the communication
// benchmark, and the one-time reset of a fresh slot.
//
// The synthetic expert is the one the reference validates with
// (benchmarks/replay.py:67-71): every received row is scaled by the sum, over
// the slots whose expert lives on this rank, of weight * per-expert factor.
// The scale is accumulated in FP32 in slot order with separately rounded
// multiply and add so that a CPU oracle reproduces it bit for bit.
#include <cuda_bf16.h>
#include "epx_device.cuh"
#include "epx_launch.h"

namespace epx {
namespace {

__global__ void __launch_bounds__(256) scale_rows_kernel(const unsigned short* __restrict__ hidden,
                                                         const long long* __restrict__ local_ids,
                                                         const float* __restrict__ weights,
                                                         const int* __restrict__ valid_count,
                                                         const float* __restrict__ factors, int num_factors,
                                                         unsigned short* __restrict__ partial, int capacity,
                                                         int hidden_size, int topk) {
  const int valid = min(*valid_count, capacity);
  const int warps_per_cta = blockDim.x / 32;
  const int lane = threadIdx.x & 31;
  const bool vec = (hidden_size % 8 == 0) && (reinterpret_cast<size_t>(hidden) % 16 == 0) &&
                   (reinterpret_cast<size_t>(partial) % 16 == 0);
  for (long long row = static_cast<long long>(blockIdx.x) * warps_per_cta + (threadIdx.x >> 5); row < valid;
       row += static_cast<long long>(gridDim.x) * warps_per_cta) {
    // Lanes fetch the slots in parallel (one memory round trip), then the scale is
    // accumulated in slot order from registers, so the arithmetic stays sequential.
    float scale = 0.f;
    for (int k0 = 0; k0 < topk; k0 += 32) {
      const int k = k0 + lane;
      float term = 0.f;
      bool local = false;
      if (k < topk) {
        const long long id = local_ids[row * topk + k];
        if (id >= 0) {
          const float f = factors != nullptr ? factors[id < num_factors ? id : num_factors - 1] : 1.f;
          term = __fmul_rn(weights[row * topk + k], f);
          local = true;
        }
      }
      const unsigned votes = __ballot_sync(0xffffffffu, local);
      const int span = min(32, topk - k0);
      for (int j = 0; j < span; ++j) {
        const float t = __shfl_sync(0xffffffffu, term, j);
        if ((votes >> j) & 1u) scale = __fadd_rn(scale, t);
      }
    }
    const unsigned short* src = hidden + row * hidden_size;
    unsigned short* dst = partial + row * hidden_size;
    if (vec) {
      constexpr int kUnroll = 8;   // 128 bytes per lane in flight: the kernel is a pure HBM stream, bound by latency
      for (int base = lane * 8; base < hidden_size; base += 32 * 8 * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int i = base + u * 256;
          if (i < hidden_size) v[u] = *reinterpret_cast<const uint4*>(src + i);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int i = base + u * 256;
          if (i >= hidden_size) continue;
          unsigned* w = reinterpret_cast<unsigned*>(&v[u]);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float lo = __fmul_rn(__uint_as_float(w[q] << 16), scale);
            const float hi = __fmul_rn(__uint_as_float(w[q] & 0xffff0000u), scale);
            w[q] = pack_bf16x2(lo, hi);
          }
          *reinterpret_cast<uint4*>(dst + i) = v[u];
        }
      }
    } else {
      for (int i = lane; i < hidden_size; i += 32)
        dst[i] = float_to_bf16_bits(__fmul_rn(bf16_bits_to_float(src[i]), scale));
    }
  }
}

__global__ void __launch_bounds__(256) slot_reset_kernel(char* slot, SlotLayout l, long long capacity, int hidden,
                                                         int topk) {
  const long long threads = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long me = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  unsigned* hid = reinterpret_cast<unsigned*>(slot + l.hidden);
  unsigned* part = reinterpret_cast<unsigned*>(slot + l.partial);
  const long long words = capacity * hidden / 2;
  for (long long i = me; i < words; i += threads) { hid[i] = 0u; part[i] = 0u; }
  long long* ids = reinterpret_cast<long long*>(slot + l.ids);
  float* w = reinterpret_cast<float*>(slot + l.weights);
  for (long long i = me; i < capacity * topk; i += threads) { ids[i] = -1; w[i] = 0.f; }
  long long* inv = reinterpret_cast<long long*>(slot + l.inverse);
  for (long long i = me; i < capacity * 2; i += threads) inv[i] = -1;
  // Arrival words behind the staging rows must never equal a combine epoch by accident (a
  // re-used heap range holds old payload): the whole plane starts at zero.
  uint4* stage = reinterpret_cast<uint4*>(slot + l.staging);
  const long long stage_vecs = static_cast<long long>(l.partial - l.staging) / 16;
  for (long long i = me; i < stage_vecs; i += threads) stage[i] = make_uint4(0u, 0u, 0u, 0u);
  unsigned* local = reinterpret_cast<unsigned*>(slot + l.mask);
  const long long local_words = static_cast<long long>(l.output - l.mask) / 4;
  for (long long i = me; i < local_words; i += threads) local[i] = 0u;
}

}  // namespace

cudaError_t launch_scale_rows(const void* hidden, const long long* local_ids, const float* weights,
                              const int* valid_count, const float* factors, int num_factors, void* partial,
                              int capacity, int hidden_size, int topk, cudaStream_t stream) {
  if (capacity <= 0) return cudaSuccess;
  const int ctas = capacity < 8 * 148 * 8 ? (capacity + 7) / 8 : 148 * 8;
  scale_rows_kernel<<<ctas, 256, 0, stream>>>(static_cast<const unsigned short*>(hidden), local_ids, weights,
                                              valid_count, factors, num_factors,
                                              static_cast<unsigned short*>(partial), capacity, hidden_size, topk);
  return cudaGetLastError();
}

cudaError_t launch_slot_reset(char* slot, SlotLayout layout, long long capacity, int hidden, int topk,
                              cudaStream_t stream) {
  slot_reset_kernel<<<148 * 4, 256, 0, stream>>>(slot, layout, capacity, hidden, topk);
  return cudaGetLastError();
}

}  // namespace epx
