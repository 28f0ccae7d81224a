// Device-side primitives shared by the transport kernels: system-scope flag
// words, bounded waits, sticky error reporting and a bounded grid barrier.
//
// The reference's equivalents are system-scope loads/stores on mapped host
// pages (ep_xpress/csrc/host_sm.cu:98-124) and a sticky status word
// (host_sm.cu:523-532). Here the words live in the RECEIVER's HBM: writers
// store across NVLink, readers poll local memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "epx_layout.h"

namespace epx {

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// Monotone publication: the word only ever grows, whichever writer's update lands last.
__device__ __forceinline__ void red_max_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("red.release.sys.global.max.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_add_relaxed_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_u32(unsigned* p, unsigned v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_volatile_i32(const int* p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_volatile_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// 16-byte payload accesses. Peer rows are rewritten every generation, so they
// must not be served from a stale L1 line: no-allocate loads after the acquire.
__device__ __forceinline__ uint4 ld_payload16(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_payload4(const void* p) {
  unsigned v;
  asm volatile("ld.global.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_payload16(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_payload4(void* p, unsigned v) {
  asm volatile("st.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ unsigned long long tagged(unsigned generation, unsigned value) {
  return (static_cast<unsigned long long>(generation) << 32) | value;
}
__device__ __forceinline__ unsigned tag_of(unsigned long long word) { return static_cast<unsigned>(word >> 32); }
__device__ __forceinline__ unsigned value_of(unsigned long long word) { return static_cast<unsigned>(word); }

__device__ __forceinline__ CtrlHeader* header_of(char* heap) { return reinterpret_cast<CtrlHeader*>(heap); }

// Record the first error, raise the local bail-out flag and tell every peer,
// so that their bounded waits end early with kPeerAbort instead of a timeout.
// (Behaviour of the arena header error word, ep_xpress/csrc/host_sm.cu:1184-1190,
// without the trap.)
static __device__ __noinline__ void report_error(const RankCtx& c, int code, unsigned phase, unsigned where,
                                          unsigned value) {
  CtrlHeader* h = header_of(c.heap[c.rank]);
  if (atomicCAS(&h->status, 0, code) == 0) {
    h->error_detail = (static_cast<unsigned long long>(phase) << 56) |
                      (static_cast<unsigned long long>(where & 0xffffffu) << 32) | value;
    const CtrlLayout l = ctrl_layout(c.world);
    for (int p = 0; p < c.world; ++p) {
      if (p == c.rank) continue;
      unsigned* slot = reinterpret_cast<unsigned*>(c.heap[p] + l.perr) + c.rank;
      st_relaxed_sys_u32(slot, static_cast<unsigned>(code));
    }
  }
  atomicExch(&h->abort_flag, 1);
  __threadfence();
}

// Poll `ready()` until it holds, the timeout passes, the local bail-out flag is
// raised or a peer published an error. Returns true only when `ready()` held.
// Never traps, never spins forever: on failure the caller unwinds and returns.
template <typename Ready>
__device__ __forceinline__ bool bounded_wait(const RankCtx& c, unsigned phase, unsigned where, Ready ready,
                                             unsigned long long* polls = nullptr) {
  if (ready()) return true;
  CtrlHeader* h = header_of(c.heap[c.rank]);
  const CtrlLayout l = ctrl_layout(c.world);
  const unsigned* perr = reinterpret_cast<const unsigned*>(c.heap[c.rank] + l.perr);
  const unsigned long long start = global_timer_ns();
  unsigned spins = 0;
  while (true) {
    if (ready()) {
      if (polls != nullptr) *polls += spins;
      return true;
    }
    if ((++spins & 63u) == 0) {
      if (ld_volatile_i32(&h->abort_flag) != 0) return false;
      for (int p = 0; p < c.world; ++p) {
        if (p != c.rank && ld_volatile_u32(perr + p) != 0) {
          report_error(c, kPeerAbort, phase, where, static_cast<unsigned>(p));
          return false;
        }
      }
      if (global_timer_ns() - start > c.timeout_ns) {
        report_error(c, kTimeout, phase, where, spins);
        return false;
      }
      __nanosleep(32);
    }
  }
}

// Barrier over the CTAs of ONE rank (blockIdx.x dimension). `target` is the
// arrival count that completes it: k * gridDim.x for the k-th barrier of the
// launch; the last CTA of the launch puts the counter back to zero. Requires a
// cooperative launch (all CTAs resident). Returns false when the rank is
// bailing out; the caller must then skip to its exit path.
__device__ __forceinline__ bool rank_barrier(const RankCtx& c, unsigned* counter, unsigned target,
                                             unsigned phase) {
  __shared__ int barrier_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
    const bool ok = bounded_wait(c, phase, 0xB0u, [&] { return ld_acquire_gpu_u32(counter) >= target; });
    __threadfence();
    barrier_ok = ok ? 1 : 0;
  }
  __syncthreads();
  return barrier_ok != 0;
}

// ---- bulk asynchronous copies (TMA, no tensor map) into this CTA's shared memory -------
__device__ __forceinline__ unsigned smem_address(const void* p) {
  return static_cast<unsigned>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbarrier_init(unsigned long long* bar, unsigned arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_address(bar)), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbarrier_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_address(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbarrier_try_wait(unsigned long long* bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(smem_address(bar)), "r"(parity) : "memory");
  return done != 0;
}
// Waits for the phase with `parity` of an mbarrier, at most `timeout_ns` on the GPU's global
// timer. Returns false when it gave up; the caller then unwinds and reports an error.
__device__ __forceinline__ bool mbarrier_wait_bounded(unsigned long long* bar, unsigned parity,
                                                      unsigned long long timeout_ns) {
  if (mbarrier_try_wait(bar, parity)) return true;
  const unsigned long long start = global_timer_ns();
  unsigned spins = 0;
  while (!mbarrier_try_wait(bar, parity))
    if ((++spins & 255u) == 0 && global_timer_ns() - start > timeout_ns) return false;
  return true;
}
// Global -> shared copy of `bytes` (a multiple of 16, both addresses 16-byte aligned) that
// signals `bar` with its byte count when the data has landed. Destination is this CTA's own
// shared memory; one copy per call, no fan-out.
__device__ __forceinline__ void bulk_load_to_smem(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_address(dst)), "l"(src), "r"(bytes), "r"(smem_address(bar)) : "memory");
}
// Orders earlier generic-proxy accesses of this thread before later async-proxy (bulk copy) ones.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Debugging aid that shakes the interleaving of ranks and CTAs: thread 0 of the CTA sleeps for a
// pseudo-random time below RankCtx::debug_delay_ns (a hash of rank, CTA, call site and the
// clock), then the CTA proceeds together. Off (zero) it costs one uniform branch. The results
// of every operation must not depend on it; the tests run the oracle comparison with it on.
__device__ __forceinline__ void debug_delay(const RankCtx& c, unsigned site) {
  if (c.debug_delay_ns == 0) return;
  if (threadIdx.x == 0) {
    unsigned h = (static_cast<unsigned>(c.rank) * 2654435761u) ^ (blockIdx.x * 40503u) ^ (site * 2246822519u) ^
                 static_cast<unsigned>(global_timer_ns() >> 5);
    h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
    const unsigned long long until = global_timer_ns() + h % c.debug_delay_ns;
    while (global_timer_ns() < until) __nanosleep(200);
  }
  __syncthreads();
}

// Profile record of this CTA (kProfileStamps words) in a profiling launch. The transport
// kernels are templates on `kProfile`: their ordinary specialisation contains none of this.
template <bool kProfile>
struct Profiler {
  unsigned long long* record;
  unsigned long long polls;     // per thread, flushed at the end
  unsigned long long rows, bytes;
  __device__ __forceinline__ explicit Profiler(unsigned long long* base)
      : record(kProfile && base != nullptr ? base + static_cast<size_t>(blockIdx.x) * kProfileStamps : nullptr),
        polls(0), rows(0), bytes(0) {}
  __device__ __forceinline__ bool on() const { return kProfile && record != nullptr; }
  // Phase stamp by thread 0 of the CTA.
  __device__ __forceinline__ void stamp(int index) const {
    if (!kProfile) return;
    if (record != nullptr && threadIdx.x == 0) {
      record[index] = global_timer_ns();
      record[kProfCompletion] = static_cast<unsigned long long>(index);
    }
  }
  __device__ __forceinline__ unsigned long long* poll_counter() { return on() ? &polls : nullptr; }
  __device__ __forceinline__ void moved(unsigned long long n_rows, unsigned long long n_bytes) {
    if (!kProfile) return;
    rows += n_rows;
    bytes += n_bytes;
  }
  // First time anything happened (any thread): keeps the earliest non-zero value.
  __device__ __forceinline__ void first(int word) const {
    if (!kProfile) return;
    if (record != nullptr) atomicCAS(record + word, 0ull, global_timer_ns());
  }
  __device__ __forceinline__ void count(int word, unsigned long long n) const {
    if (!kProfile) return;
    if (record != nullptr && n != 0) atomicAdd(record + word, n);
  }
  // Called by every thread on its way out.
  __device__ __forceinline__ void flush(const int* status) const {
    if (!kProfile) return;
    if (record == nullptr) return;
    if (rows) atomicAdd(record + kProfRows, rows);
    if (bytes) atomicAdd(record + kProfBytes, bytes);
    if (polls) atomicAdd(record + kProfPolls, polls);
    if (threadIdx.x == 0) record[kProfStatus] = static_cast<unsigned long long>(ld_volatile_i32(status));
  }
};

// Sample ring of graph-replayed operations (layout: kSampleWords in epx_layout.h). Returns the
// sample index of the operation with `generation`, or ~0u when nothing is to be recorded;
// thread 0 of every CTA offers its start time. An operation beyond the ring's capacity only
// counts itself as dropped (once, by CTA 0).
__device__ __forceinline__ unsigned sample_begin(unsigned long long* ring, unsigned generation, int capacity) {
  if (ring == nullptr || threadIdx.x != 0) return ~0u;
  if (ld_relaxed_sys(ring + 2) == 0ull) return ~0u;
  const unsigned index = generation - static_cast<unsigned>(ld_relaxed_sys(ring + 1));
  if (index < static_cast<unsigned>(capacity)) {
    atomicMin(ring + static_cast<size_t>(1 + index) * kSampleWords, global_timer_ns());
    return index;
  }
  if (blockIdx.x == 0 && static_cast<int>(index) >= capacity) atomicAdd(ring, 1ull);
  return ~0u;
}
__device__ __forceinline__ void sample_end(unsigned long long* ring, unsigned index) {
  if (index == ~0u) return;
  unsigned long long* row = ring + static_cast<size_t>(1 + index) * kSampleWords;
  atomicMax(row + 1, global_timer_ns());
  atomicAdd(row + 2, 1ull);
}

__device__ __forceinline__ float bf16_bits_to_float(unsigned short bits) {
  return __uint_as_float(static_cast<unsigned>(bits) << 16);
}
__device__ __forceinline__ unsigned short float_to_bf16_bits(float v) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
// Two floats rounded (to nearest even) and packed as one BF16 pair in a single instruction;
// `lo` becomes the low half, i.e. the element at the lower address.
__device__ __forceinline__ unsigned pack_bf16x2(float lo, float hi) {
  unsigned d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
// Pairs of floats in one 64-bit register for the packed FP32 adder of sm_100: the reduce loops
// are bound by instruction issue, and one add.rn.f32x2 does the work of two FADDs with the same
// IEEE result per element.
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
  unsigned long long d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long add_f32x2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ unsigned long long bf16x2_to_f32x2(unsigned pair) {
  return pack_f32x2(__uint_as_float(pair << 16), __uint_as_float(pair & 0xffff0000u));
}

}  // namespace epx
