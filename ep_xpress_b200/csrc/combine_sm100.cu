// Fused expert-parallel combine for sm_100a. Every expert rank PUSHES its
// already-weighted partial rows straight into the staging plane of the rank that
// owns the token (peer stores over NVLink, the direction that runs at link
// speed; peer loads do not), signals, and every source rank then reduces its
// tokens in one pass:
//
//   out[t] = bf16( float( bf16( sum_{r != self, ascending r} float(partial_r[t]) ) )
//                  + float(partial_self[t]) )
//
// i.e. remote ranks are accumulated in FP32 in ascending rank order starting
// from +0, rounded to BF16, then the local contribution is added and the sum is
// rounded again - the arithmetic of the reference's finalize/reduce kernels
// (ep_xpress/csrc/kernels.cu:27-36, ep_xpress/csrc/host_sm.cu:592-607 and
// :1846-1895). RankCtx::single_round selects the multi-node variant instead:
// one FP32 accumulation over all contributing ranks in rank order and a single
// rounding (ep_xpress/csrc/gin.cu:226-246). Arrival order never changes the
// arithmetic: a token's contributions sit at fixed staging rows (token * fanout
// + j, j-th destination rank ascending) and are added in that order.
//
// One launch replaces the reference's zero-fill, pair transport and reduce
// launches (host_sm.cu:559-590, :1212-1468, :592-607). Protocol:
//   A. push    work items (received row, row segment) claimed from a local counter:
//              rows whose source is a peer are stored to that peer's staging plane
//              at the return slot the dispatch recorded next to the row;
//   B. signal  the last CTA publishes the monotone combine epoch to every peer
//              after a system fence;
//   C. wait    bounded, for the epoch of exactly the peers this rank sent rows to;
//   D. reduce  work items (token, segment): staging rows and the local partial row
//              are read from this GPU's own memory and reduced in rank order;
//   E. retire  the last CTA advances the device epoch.
// No trailing handshake is needed: a staging plane is only rewritten by the combine
// of a later dispatch on the same slot, which cannot complete before this rank has
// entered that dispatch, i.e. finished this reduce.
#include "epx_device.cuh"
#include "epx_launch.h"

namespace epx {
namespace {

constexpr unsigned kPhaseCombine = 2;
constexpr int kPeerBatch = 8;   // peer rows whose loads are in flight together

template <int kWords>
struct Chunk {
  unsigned w[kWords];
};

template <int kWords>
__device__ __forceinline__ Chunk<kWords> load_chunk(const char* p) {
  Chunk<kWords> c;
  if (kWords == 4) {
    const uint4 v = ld_payload16(p);
    c.w[0] = v.x; c.w[1 % kWords] = v.y; c.w[2 % kWords] = v.z; c.w[3 % kWords] = v.w;
  } else {
    c.w[0] = ld_payload4(p);
  }
  return c;
}

template <int kWords>
__device__ __forceinline__ Chunk<kWords> load_local_chunk(const char* p) {
  Chunk<kWords> c;
  if (kWords == 4) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    c.w[0] = v.x; c.w[1 % kWords] = v.y; c.w[2 % kWords] = v.z; c.w[3 % kWords] = v.w;
  } else {
    c.w[0] = *reinterpret_cast<const unsigned*>(p);
  }
  return c;
}

template <int kWords>
__device__ __forceinline__ void store_chunk(char* p, const Chunk<kWords>& c) {
  if (kWords == 4) st_payload16(p, make_uint4(c.w[0], c.w[1 % kWords], c.w[2 % kWords], c.w[3 % kWords]));
  else st_payload4(p, c.w[0]);
}

template <int kWords>
__device__ __forceinline__ void accumulate(float* acc, const Chunk<kWords>& c) {
#pragma unroll
  for (int i = 0; i < kWords; ++i) {
    acc[2 * i] = __fadd_rn(acc[2 * i], __uint_as_float(c.w[i] << 16));
    acc[2 * i + 1] = __fadd_rn(acc[2 * i + 1], __uint_as_float(c.w[i] & 0xffff0000u));
  }
}

// Two-step rounding (default) or single rounding of the accumulated sum.
template <int kWords>
__device__ __forceinline__ Chunk<kWords> finish(const float* acc, const Chunk<kWords>& local, bool has_local,
                                                bool single_round) {
  Chunk<kWords> out;
#pragma unroll
  for (int i = 0; i < kWords; ++i) {
    float lo = acc[2 * i], hi = acc[2 * i + 1];
    if (!single_round) {
      const float llo = has_local ? __uint_as_float(local.w[i] << 16) : 0.f;
      const float lhi = has_local ? __uint_as_float(local.w[i] & 0xffff0000u) : 0.f;
      lo = __fadd_rn(bf16_bits_to_float(float_to_bf16_bits(lo)), llo);
      hi = __fadd_rn(bf16_bits_to_float(float_to_bf16_bits(hi)), lhi);
    }
    out.w[i] = static_cast<unsigned>(float_to_bf16_bits(lo)) |
               (static_cast<unsigned>(float_to_bf16_bits(hi)) << 16);
  }
  return out;
}

// Reduce one row segment whose contributors' row pointers sit in registers:
// kPeers rows x kUnroll chunks of loads are issued before the first add; adds
// then run in ascending rank order per chunk.
struct RowPointers {
  const char* row[kPeerBatch];
};

template <int kWords, int kPeers, int kUnroll>
__device__ __noinline__ void reduce_rows(RowPointers rows, const char* local_ptr, char* outp, long long b0,
                                         long long b1, int lane, bool single_round) {
  constexpr int kChunk = kWords * 4;
  const char* const* rp = rows.row;
  for (long long base = b0 + static_cast<long long>(lane) * kChunk; base < b1; base += 32ll * kChunk * kUnroll) {
    Chunk<kWords> v[kPeers][kUnroll];
    Chunk<kWords> local[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long off = base + static_cast<long long>(u) * 32 * kChunk;
      if (off < b1) {
#pragma unroll
        for (int b = 0; b < kPeers; ++b)
          if (rp[b] != nullptr) v[b][u] = load_chunk<kWords>(rp[b] + off);
        if (local_ptr != nullptr) local[u] = load_local_chunk<kWords>(local_ptr + off);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long off = base + static_cast<long long>(u) * 32 * kChunk;
      if (off < b1) {
        float acc[kWords * 2];
#pragma unroll
        for (int i = 0; i < kWords * 2; ++i) acc[i] = 0.f;
#pragma unroll
        for (int b = 0; b < kPeers; ++b)
          if (rp[b] != nullptr) accumulate<kWords>(acc, v[b][u]);
        store_chunk<kWords>(outp + off, finish<kWords>(acc, local[u], local_ptr != nullptr, single_round));
      }
    }
  }
}

// More contributors than registers (groups wider than kPeerBatch ranks): batches of
// kPeerBatch loads, still added in ascending rank order. Lane j holds the pointer of
// contributor j (ptr_a) and j + 32 (ptr_b).
template <int kWords>
__device__ __noinline__ void reduce_rows_generic(const char* ptr_a, const char* ptr_b, int n, int skip,
                                                 const char* local_ptr, char* outp, long long b0, long long b1,
                                                 int lane, bool single_round) {
  constexpr int kChunk = kWords * 4;
  for (long long batch = b0; batch < b1; batch += 32ll * kChunk) {   // warp-uniform trip count
    const long long off = batch + static_cast<long long>(lane) * kChunk;
    const bool active = off < b1;
    float acc[kWords * 2];
#pragma unroll
    for (int i = 0; i < kWords * 2; ++i) acc[i] = 0.f;
    for (int j0 = 0; j0 < n; j0 += kPeerBatch) {
      Chunk<kWords> v[kPeerBatch];
      bool use[kPeerBatch];
#pragma unroll
      for (int b = 0; b < kPeerBatch; ++b) {
        const int j = j0 + b;
        const unsigned long long bits =
            __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(j < 32 ? ptr_a : ptr_b), j & 31);
        use[b] = active && j < n && j != skip && bits != 0ull;
        if (use[b]) v[b] = load_chunk<kWords>(reinterpret_cast<const char*>(bits) + off);
      }
#pragma unroll
      for (int b = 0; b < kPeerBatch; ++b)
        if (use[b]) accumulate<kWords>(acc, v[b]);
    }
    if (active) {
      Chunk<kWords> local;
      if (local_ptr != nullptr) local = load_chunk<kWords>(local_ptr + off);
      store_chunk<kWords>(outp + off, finish<kWords>(acc, local, local_ptr != nullptr, single_round));
    }
  }
}

__device__ __forceinline__ int nth_set_bit(unsigned long long mask, int n) {
  for (int i = 0; i < n; ++i) mask &= mask - 1;
  return __ffsll(static_cast<long long>(mask)) - 1;
}

// ---- reduce phase, bulk-copy variant (rows 16-byte aligned) -------------------------------
// Each warp streams its work item through a ring of shared-memory stages: lanes that hold a
// contributor's row pointer issue one bulk copy (TMA) of the next 512-byte step of that row,
// all contributors of a step complete on one mbarrier, and the warp then adds the staged
// chunks in ascending rank order. Data in flight lives in shared memory, not in registers,
// so the phase runs at memory speed with a small register footprint.
constexpr int kStepBytes = 512;                 // 32 lanes x 16 bytes
constexpr int kStages = 3;
constexpr int kStageBytes = kPeerBatch * kStepBytes;
constexpr int kWarpRingBytes = kStages * kStageBytes;
constexpr int kCombineWarps = kThreads / 32;
constexpr size_t kCombineSmemBytes = static_cast<size_t>(kCombineWarps) * kWarpRingBytes;
constexpr unsigned kMbarrierSpinLimit = 1u << 24;

struct WarpRing {
  char* buffer;                    // kStages x kPeerBatch x kStepBytes of this warp
  unsigned long long* bars;        // kStages mbarriers of this warp
  unsigned issued;                 // units issued so far (persist across work items)
  unsigned consumed;               // units consumed so far
};

// A unit is (step of the row segment, batch of up to kPeerBatch contributors).
__device__ __forceinline__ void ring_issue(WarpRing& ring, const char* ptr_a, const char* ptr_b, int n, int batch,
                                           long long offset, unsigned bytes, int lane) {
  const int stage = ring.issued % kStages;
  const int first = batch * kPeerBatch;                 // first contributor of this batch
  const int local = lane - (first & 31);                // this lane's position inside the batch
  const bool mine = local >= 0 && local < kPeerBatch && first + local < n;
  const char* src = (first < 32) ? ptr_a : ptr_b;
  const bool valid = mine && src != nullptr;
  const unsigned votes = __ballot_sync(0xffffffffu, valid);
  __syncwarp();                                         // everyone finished reading this stage
  if (lane == 0) {
    fence_proxy_async();
    mbarrier_arrive_expect_tx(ring.bars + stage, static_cast<unsigned>(__popc(votes)) * bytes);
  }
  __syncwarp();
  if (valid) bulk_load_to_smem(ring.buffer + stage * kStageBytes + local * kStepBytes, src + offset, bytes,
                               ring.bars + stage);
  ++ring.issued;
}

__device__ __forceinline__ bool ring_wait(WarpRing& ring) {
  const int stage = ring.consumed % kStages;
  const unsigned parity = (ring.consumed / kStages) & 1u;
  unsigned spins = 0;
  while (!mbarrier_try_wait(ring.bars + stage, parity))
    if (++spins > kMbarrierSpinLimit) return false;
  return true;
}

// Reduce one row segment [b0, b1) of token t. Lane j holds contributor j (ptr_a) and j + 32
// (ptr_b), ascending rank order; self_index is this rank's own position or -1.
__device__ __forceinline__ bool reduce_segment_bulk(WarpRing& ring, const char* ptr_a, const char* ptr_b, int n,
                                                    int self_index, bool single_round, char* outp, long long b0,
                                                    long long b1, int lane) {
  const int batches = n == 0 ? 0 : (n + kPeerBatch - 1) / kPeerBatch;
  const int steps = static_cast<int>((b1 - b0 + kStepBytes - 1) / kStepBytes);
  if (batches == 0) {                                   // padding token: zero row
    for (long long off = b0 + lane * 16; off < b1; off += kStepBytes) st_payload16(outp + off, make_uint4(0, 0, 0, 0));
    return true;
  }
  const unsigned valid_a = __ballot_sync(0xffffffffu, ptr_a != nullptr);
  const unsigned valid_b = __ballot_sync(0xffffffffu, ptr_b != nullptr);
  const int units = steps * batches;
  int issued = 0;
  auto issue_next = [&]() {
    const int step = issued / batches, batch = issued % batches;
    const long long offset = b0 + static_cast<long long>(step) * kStepBytes;
    const unsigned bytes = static_cast<unsigned>(min(static_cast<long long>(kStepBytes), b1 - offset));
    ring_issue(ring, ptr_a, ptr_b, n, batch, offset, bytes, lane);
    ++issued;
  };
  for (int u = 0; u < kStages - 1 && issued < units; ++u) issue_next();
  float acc[8];
  Chunk<4> local;
  bool has_local = false;
  for (int unit = 0; unit < units; ++unit) {
    const int step = unit / batches, batch = unit % batches;
    if (issued < units) issue_next();
    if (!ring_wait(ring)) return false;
    const long long offset = b0 + static_cast<long long>(step) * kStepBytes;
    const bool active = offset + lane * 16 < b1;
    if (batch == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      has_local = false;
    }
    const char* stage = ring.buffer + (ring.consumed % kStages) * kStageBytes + lane * 16;
    const int first = batch * kPeerBatch;
    const unsigned valid = (first < 32 ? valid_a : valid_b) >> (first & 31);
#pragma unroll
    for (int i = 0; i < kPeerBatch; ++i) {
      if (first + i < n && ((valid >> i) & 1u) && active) {
        const uint4 v = *reinterpret_cast<const uint4*>(stage + i * kStepBytes);
        Chunk<4> c;
        c.w[0] = v.x; c.w[1] = v.y; c.w[2] = v.z; c.w[3] = v.w;
        if (!single_round && first + i == self_index) {
          local = c;
          has_local = true;
        } else {
          accumulate<4>(acc, c);
        }
      }
    }
    ++ring.consumed;
    if (batch == batches - 1 && active)
      store_chunk<4>(outp + offset + lane * 16, finish<4>(acc, local, has_local, single_round));
  }
  return true;
}

template <bool kVec16>
__device__ __forceinline__ void combine_body(const CombineOp& op, char* dynamic_smem) {
  constexpr int kWords = kVec16 ? 4 : 1;
  constexpr int kChunk = kWords * 4;
  constexpr int kUnroll = 4;
  const RankCtx& c = *op.ctx;
  const int W = c.world, self = c.rank, H = c.hidden, K = c.topk;
  const bool single_round = c.single_round != 0;
  const int tid = threadIdx.x, lane = tid & 31;
  const int T = op.tokens;
  char* const my_heap = c.heap[self];
  CtrlHeader* const hdr = header_of(my_heap);
  const CtrlLayout cl = ctrl_layout(W);
  const SlotLayout sl = slot_layout(op.slot_capacity, op.slot_tokens, H, K, W);
  char* const slot = my_heap + op.slot_off;
  const unsigned long long* const mask_arr = reinterpret_cast<const unsigned long long*>(slot + sl.mask);
  const int* const send_rows = reinterpret_cast<const int*>(slot + sl.send_rows);
  const long long* const inverse = reinterpret_cast<const long long*>(slot + sl.inverse);
  const int* const ret = reinterpret_cast<const int*>(slot + sl.ret);
  const int* const misc = reinterpret_cast<const int*>(slot + sl.misc);
  const char* const partial = reinterpret_cast<const char*>(op.partial);
  const char* const staging = slot + sl.staging;
  const int fan = route_fanout(K, W);
  const long long row_bytes = static_cast<long long>(H) * 2;

  __shared__ char* s_stage[64];
  __shared__ int s_need[64];
  __shared__ int s_last;

  profile_stamp(op.profile, 0);
  const unsigned e = ld_volatile_u32(&hdr->comb_epoch) + 1;
  if (tid < W) {
    const unsigned long long off = reinterpret_cast<const unsigned long long*>(slot + sl.peer_off)[tid];
    const int cap = reinterpret_cast<const int*>(slot + sl.peer_cap)[tid];
    const SlotLayout pl = slot_layout(cap, 0, H, K, W);
    s_stage[tid] = c.heap[tid] + off + pl.staging;
    s_need[tid] = (tid != self && reinterpret_cast<const int*>(slot + sl.send_cnt)[tid] > 0) ? 1 : 0;
  }
  const int valid = min(misc[kValidCount], op.partial_rows);
  const int segs = op.segments;
  const long long seg_bytes = align_up((row_bytes + segs - 1) / segs, 32 * kChunk * kUnroll);
  __syncthreads();

  // ---- A. push my rows to the ranks that own the tokens ---------------------------
  {
    const long long items = static_cast<long long>(valid) * segs;
    while (true) {
      unsigned claimed = 0;
      if (lane == 0) claimed = atomicAdd(&hdr->cwork_push, 1u);
      const long long item = __shfl_sync(0xffffffffu, claimed, 0);
      if (item >= items) break;
      const long long row = item / segs;
      const int seg = static_cast<int>(item % segs);
      const int source = static_cast<int>(inverse[row * 2]);
      if (source == self || source < 0 || source >= W) continue;
      const long long back = ret[row];
      const char* src = partial + row * row_bytes;
      char* dst = s_stage[source] + back * row_bytes;
      const long long b0 = seg * seg_bytes;
      const long long b1 = min(row_bytes, b0 + seg_bytes);
      for (long long base = b0 + static_cast<long long>(lane) * kChunk; base < b1; base += 32ll * kChunk * kUnroll) {
        Chunk<kWords> v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const long long off = base + static_cast<long long>(u) * 32 * kChunk;
          if (off < b1) v[u] = load_local_chunk<kWords>(src + off);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const long long off = base + static_cast<long long>(u) * 32 * kChunk;
          if (off < b1) store_chunk<kWords>(dst + off, v[u]);
        }
      }
    }
  }
  __syncthreads();
  profile_stamp(op.profile, 1);

  // ---- B. signal ------------------------------------------------------------------------
  if (tid == 0) {
    __threadfence_system();
    const unsigned prev = atomicAdd(&hdr->cdone_count, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
    if (s_last) __threadfence_system();
  }
  __syncthreads();
  if (s_last && tid < W && tid != self) {
    unsigned long long* flag = reinterpret_cast<unsigned long long*>(c.heap[tid] + cl.ready) + self;
    st_release_sys(flag, static_cast<unsigned long long>(e));
  }

  // ---- C. wait for the peers that push to me ----------------------------------------------
  bool ok = true;
  if (tid < W && s_need[tid]) {
    const unsigned long long* flag = reinterpret_cast<const unsigned long long*>(my_heap + cl.ready) + tid;
    ok = bounded_wait(c, kPhaseCombine, 2, [&] { return ld_acquire_sys(flag) >= e; });
  }
  if (!__syncthreads_and(ok)) return;
  profile_stamp(op.profile, 2);

  // ---- D. rank-order reduce from local memory -----------------------------------------------
  {
    __shared__ unsigned long long s_bars[kCombineWarps * kStages];
    WarpRing ring;
    ring.buffer = dynamic_smem + static_cast<size_t>(tid >> 5) * kWarpRingBytes;
    ring.bars = s_bars + (tid >> 5) * kStages;
    ring.issued = ring.consumed = 0;
    if (kVec16) {
      if (lane < kStages) mbarrier_init(ring.bars + lane, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      fence_proxy_async();
      __syncwarp();
    }
    bool healthy = true;
    const long long items = static_cast<long long>(T) * segs;
    while (healthy) {
      unsigned claimed = 0;
      if (lane == 0) claimed = atomicAdd(&hdr->cwork_reduce, 1u);
      const long long item = __shfl_sync(0xffffffffu, claimed, 0);
      if (item >= items) break;
      const int t = static_cast<int>(item / segs), seg = static_cast<int>(item % segs);
      const unsigned long long m = mask_arr[t];
      const int n = __popcll(m);
      const long long b0 = seg * seg_bytes;
      const long long b1 = min(row_bytes, b0 + seg_bytes);
      char* const outp = reinterpret_cast<char*>(op.out) + static_cast<long long>(t) * row_bytes;

      // Lane j (and j + 32) resolves the j-th contributor in ascending rank order.
      const char* ptr_a = nullptr;
      const char* ptr_b = nullptr;
      int self_index = -1;
      {
        bool is_self = false;
        if (lane < n) {
          const int d = nth_set_bit(m, lane);
          const int row = send_rows[static_cast<long long>(t) * fan + lane];
          is_self = (d == self);
          if (row >= 0 && !(is_self && row >= op.partial_rows))
            ptr_a = is_self ? partial + static_cast<long long>(row) * row_bytes
                            : staging + (static_cast<long long>(t) * fan + lane) * row_bytes;
        }
        const unsigned vote_a = __ballot_sync(0xffffffffu, is_self);
        is_self = false;
        if (lane + 32 < n) {
          const int d = nth_set_bit(m, lane + 32);
          const int row = send_rows[static_cast<long long>(t) * fan + lane + 32];
          is_self = (d == self);
          if (row >= 0 && !(is_self && row >= op.partial_rows))
            ptr_b = is_self ? partial + static_cast<long long>(row) * row_bytes
                            : staging + (static_cast<long long>(t) * fan + lane + 32) * row_bytes;
        }
        const unsigned vote_b = __ballot_sync(0xffffffffu, is_self);
        if (vote_a) self_index = __ffs(vote_a) - 1;
        else if (vote_b) self_index = 32 + __ffs(vote_b) - 1;
      }
      const int skip = single_round ? -1 : self_index;
      const unsigned long long local_bits =
          (self_index < 0 || single_round) ? 0ull
          : __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(self_index < 32 ? ptr_a : ptr_b), self_index & 31);
      const char* const local_ptr = reinterpret_cast<const char*>(local_bits);

      if (kVec16) {
        healthy = reduce_segment_bulk(ring, ptr_a, ptr_b, n, self_index, single_round, outp, b0, b1, lane);
      } else if (n <= kPeerBatch) {
        // Common case: every contributor's row pointer sits in a register.
        RowPointers rp;
#pragma unroll
        for (int b = 0; b < kPeerBatch; ++b) {
          const unsigned long long bits = __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(ptr_a), b);
          rp.row[b] = (b < n && b != skip) ? reinterpret_cast<const char*>(bits) : nullptr;
        }
        if (n <= 2) reduce_rows<kWords, 2, 4>(rp, local_ptr, outp, b0, b1, lane, single_round);
        else if (n <= 4) reduce_rows<kWords, 4, 2>(rp, local_ptr, outp, b0, b1, lane, single_round);
        else reduce_rows<kWords, kPeerBatch, 1>(rp, local_ptr, outp, b0, b1, lane, single_round);
      } else {
        reduce_rows_generic<kWords>(ptr_a, ptr_b, n, skip, local_ptr, outp, b0, b1, lane, single_round);
      }
    }
    if (!healthy) report_error(c, kTimeout, kPhaseCombine, 4, 0);
  }

  // ---- E. retire the epoch ---------------------------------------------------------------
  __syncthreads();
  profile_stamp(op.profile, 3);
  if (tid == 0) {
    const unsigned prev = atomicAdd(&hdr->cfin_count, 1u);
    if (prev == gridDim.x - 1) {
      hdr->cdone_count = 0;
      hdr->cfin_count = 0;
      hdr->cwork_push = 0;
      hdr->cwork_reduce = 0;
      hdr->comb_epoch = e;
      __threadfence();
    }
  }
}

template <bool kVec16>
__global__ void __launch_bounds__(kThreads, 1) combine_kernel(const __grid_constant__ CombineArgs args) {
  extern __shared__ __align__(128) char combine_smem[];
  combine_body<kVec16>(args.op[blockIdx.y], combine_smem);
}

template <bool kVec16>
cudaError_t prepare_combine_kernel(size_t* dynamic_smem) {
  *dynamic_smem = kVec16 ? kCombineSmemBytes : 0;
  if (*dynamic_smem <= 48 * 1024) return cudaSuccess;
  return cudaFuncSetAttribute(combine_kernel<kVec16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(*dynamic_smem));
}

}  // namespace

cudaError_t combine_max_ctas(bool vec16, int* ctas) {
  int device = 0, sms = 0, per_sm = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (err != cudaSuccess) return err;
  size_t smem = 0;
  err = vec16 ? prepare_combine_kernel<true>(&smem) : prepare_combine_kernel<false>(&smem);
  if (err != cudaSuccess) return err;
  err = vec16 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, combine_kernel<true>, kThreads, smem)
              : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, combine_kernel<false>, kThreads, smem);
  if (err != cudaSuccess) return err;
  *ctas = per_sm * sms;
  return cudaSuccess;
}

cudaError_t launch_combine(const CombineArgs& args, int ranks, int ctas_per_rank, bool vec16, bool cooperative,
                           cudaStream_t stream) {
  void* params[] = {const_cast<CombineArgs*>(&args)};
  size_t smem = 0;
  cudaError_t err = vec16 ? prepare_combine_kernel<true>(&smem) : prepare_combine_kernel<false>(&smem);
  if (err != cudaSuccess) return err;
  const void* kernel = vec16 ? reinterpret_cast<const void*>(combine_kernel<true>)
                             : reinterpret_cast<const void*>(combine_kernel<false>);
  if (!cooperative)
    return cudaLaunchKernel(kernel, dim3(ctas_per_rank, ranks, 1), dim3(kThreads, 1, 1), params, smem, stream);
  return cudaLaunchCooperativeKernel(kernel, dim3(ctas_per_rank, ranks, 1), dim3(kThreads, 1, 1), params, smem, stream);
}

}  // namespace epx
