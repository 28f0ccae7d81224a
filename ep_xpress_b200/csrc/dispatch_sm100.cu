// Fused expert-parallel dispatch for sm_100a: top-k routing, one-row-per-
// destination-rank dedup, per-rank counts and offset prefix sums, and the BF16
// payload pack, with the rows stored straight into the destination ranks'
// receive tensors over NVLink (plain peer stores; local rows take the same
// path into the rank's own heap). No staging buffer, no per-op host work, no
// cross-GPU atomics.
//
// What the reference does with a persistent host-ring kernel plus init and
// finalize launches (ep_xpress/csrc/host_sm.cu:559-607 and :613-1191) is one
// launch here:
//   1. route     every CTA maps a tile of tokens to a 64-bit destination mask
//                (dedup), validates ids/weights, and counts rows per destination;
//   2. publish   after one rank-local barrier the rank's count row goes to every
//                peer as generation-tagged words (this message is also the
//                credit "my receive slot of this generation is free");
//   3. offsets   once all count rows are in, every rank knows
//                offset[self->d] = sum_{s<self} count[s->d] and valid_count[d];
//                rows therefore land in (source rank, token) order, the order of
//                the reference's CPU planner (ep_xpress/routing.py:140-158);
//   4. payload   four mover warps per CTA claim tokens; a row is read ONCE into shared
//                memory by a bulk asynchronous copy (TMA, no tensor map) and stored
//                from there to every destination rank's plane by bulk copies, local
//                and peer alike - the first loads are already in flight while the
//                counts are awaited. The other warps write the translated local
//                expert ids, the weights and the (source, token) inverse entry.
//                Rows that are not 16-byte aligned take a register path;
//   5. signal    every CTA, after a system fence, counts itself in at the destinations
//                that got rows from this rank;
//   6. receive   padding rows are reset, valid_count is written, and the launch
//                ends once every sender with rows for this rank has signalled.
// Every wait is bounded by RankCtx::timeout_ns and ends in a status code.
#include "epx_device.cuh"
#include "epx_launch.h"

namespace epx {
namespace {

constexpr unsigned kPhaseDispatch = 1;
constexpr int kWarps = kThreads / 32;
constexpr int kRegK = 8;   // top-k up to which a token's ids and weights are routed from registers
constexpr int kMovers = 4;              // warps of a CTA that move payload with bulk copies
constexpr int kMoveStages = 3;          // row pieces one mover keeps in shared memory
constexpr int kMoveStageBytes = 14336;  // largest piece (a whole DeepSeek-V3 row)
constexpr size_t kMoveRingBytes = static_cast<size_t>(kMovers) * kMoveStages * kMoveStageBytes;

__device__ __forceinline__ void bulk_store_from_smem(void* dst, const void* src, unsigned bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_address(src)),
               "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// The bulk copies this thread committed have finished READING shared memory (the stage may be refilled).
__device__ __forceinline__ void bulk_wait_all_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// ... have read their source AND their writes are complete.
__device__ __forceinline__ void bulk_wait_all_complete() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

struct PeerPlanes {
  char* hidden;
  char* ids;
  char* weights;
  char* inverse;
  char* ret;
};

template <typename IdT>
__device__ __forceinline__ long long load_id(const void* ids, long long index) {
  return static_cast<long long>(reinterpret_cast<const IdT*>(ids)[index]);
}

__device__ __forceinline__ int nth_set_bit(unsigned long long mask, int n) {
  for (int i = 0; i < n; ++i) mask &= mask - 1;
  return __ffsll(static_cast<long long>(mask)) - 1;
}

template <typename IdT, bool kVec16, bool kProfile>
__device__ __forceinline__ void dispatch_body(const DispatchOp& op, int* tile_base) {
  const RankCtx& c = *op.ctx;
  const int W = c.world, self = c.rank, H = c.hidden, K = c.topk, E = c.num_experts;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int T = op.tokens;
  char* const my_heap = c.heap[self];
  CtrlHeader* const hdr = header_of(my_heap);
  const CtrlLayout cl = ctrl_layout(W);
  const SlotLayout sl = slot_layout(op.slot_capacity, op.slot_tokens, H, K, W);
  char* const slot = my_heap + op.slot_off;
  unsigned long long* const mask_arr = reinterpret_cast<unsigned long long*>(slot + sl.mask);
  int* const dest_rows = reinterpret_cast<int*>(slot + sl.dest_rows);
  int* const send_rows = reinterpret_cast<int*>(slot + sl.send_rows);
  int* const tile_cnt = reinterpret_cast<int*>(slot + sl.tile_cnt);
  int* const misc = reinterpret_cast<int*>(slot + sl.misc);
  const int fan = route_fanout(K, W);
  const int ntiles = route_tiles(T);

  __shared__ int s_warp_cnt[kWarps][64];
  __shared__ int s_send[64], s_off[64], s_total[64], s_ok[64], s_ctas[64];
  __shared__ char* s_heap[64];
  __shared__ PeerPlanes s_planes[64];
  __shared__ int s_last;
  __shared__ unsigned long long s_mfull[kMovers * kMoveStages];

  Profiler<kProfile> prof(op.profile);
  prof.stamp(0);
  if (prof.on() && threadIdx.x == 0) prof.record[kProfMode] = kVec16 ? 2 : 1;
  const unsigned g = ld_volatile_u32(&hdr->disp_epoch) + 1;
  // Generations never wrap (the reference stops at 2^31 too, ep_xpress/csrc/host_sm.cu:563-567):
  // every CTA reads the same header word, so all of them leave here together.
  if (g > kLastEpoch) {
    if (threadIdx.x == 0 && blockIdx.x == 0) report_error(c, kEpochsExhausted, kPhaseDispatch, 0xE0, g);
    return;
  }
  const int par = static_cast<int>(g & 1u);
  const unsigned sample = sample_begin(op.samples, g, op.sample_capacity);
  const int dirty_prev = misc[kDirtyRows];
  unsigned long long* const my_cnt = reinterpret_cast<unsigned long long*>(my_heap + cl.cnt) +
                                     static_cast<size_t>(par) * W * W;
  unsigned long long* const my_addr = reinterpret_cast<unsigned long long*>(my_heap + cl.addr) +
                                      static_cast<size_t>(par) * W * kAddrWords;
  unsigned long long* const my_done = reinterpret_cast<unsigned long long*>(my_heap + cl.done) +
                                      static_cast<size_t>(par) * W;
  if (tid < W) s_heap[tid] = c.heap[tid];
  if (kVec16 && tid >= 64 && tid < 64 + kMovers * kMoveStages) {
    mbarrier_init(s_mfull + (tid - 64), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }

  // A group of one rank exchanges nothing: its counts and its slot are known here.
  const bool lone = W == 1;
  // Credit + address: does not depend on routing, so it leaves first.
  if (blockIdx.x == 0 && tid < W && !lone) {
    unsigned long long* a = reinterpret_cast<unsigned long long*>(c.heap[tid] + cl.addr) +
                            (static_cast<size_t>(par) * W + self) * kAddrWords;
    st_relaxed_sys(a + 0, tagged(g, static_cast<unsigned>(op.slot_off >> 8)));
    st_relaxed_sys(a + 1, tagged(g, static_cast<unsigned>(op.slot_capacity)));
    st_relaxed_sys(a + 2, tagged(g, static_cast<unsigned>(op.capacity)));
    st_relaxed_sys(a + 3, tagged(g, static_cast<unsigned>(op.identity)));
    st_relaxed_sys(a + 4, tagged(g, gridDim.x));
    if (tid == 0) prof.first(kProfFirstPublish);
  }

  // ---- 1. route ------------------------------------------------------------
  // A batch of at most one tile (decode) is routed by EVERY CTA redundantly: all CTAs write
  // identical values and each reads back only what its own threads wrote before a CTA
  // barrier, so the rank-wide barrier and its round trip through L2 are skipped.
  // (Fan-outs above eight spill positions to the dest_rows plane in two steps, which CTAs that
  // run ahead of one another would overwrite with stale values: those take the barrier.)
  const bool solo = ntiles <= 1 && fan <= 8;
  for (int tile = solo ? 0 : blockIdx.x; tile < ntiles; tile += solo ? 1 : gridDim.x) {
    const int t = tile * kRouteTile + tid;
    unsigned long long m = 0;
    if (t < T) {
      bool bad = false;
      const long long row = static_cast<long long>(t) * K;
      if (K <= kRegK) {
        // Independent loads first, lookups second, checks in registers: the route phase is a
        // chain of dependent memory latencies, not bandwidth.
        long long id[kRegK];
        float w[kRegK];
        int owner[kRegK];
#pragma unroll
        for (int k = 0; k < kRegK; ++k) {
          id[k] = k < K ? load_id<IdT>(op.ids, row + k) : -1;
          w[k] = k < K ? op.weights[row + k] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < kRegK; ++k) {
          const bool in_range = id[k] >= 0 && id[k] < E;
          owner[k] = in_range ? c.expert_rank[id[k]] : -1;
          if (id[k] != -1 && (!in_range || !isfinite(w[k]))) bad = true;
        }
#pragma unroll
        for (int k = 0; k < kRegK; ++k) {
          if (owner[k] >= 0) m |= 1ull << owner[k];
#pragma unroll
          for (int j = 0; j < k; ++j)
            if (id[k] >= 0 && id[j] == id[k]) bad = true;
        }
      } else {
        for (int k = 0; k < K; ++k) {
          const long long id = load_id<IdT>(op.ids, row + k);
          if (id == -1) continue;
          if (id < 0 || id >= E) { bad = true; continue; }
          const float w = op.weights[row + k];
          if (!isfinite(w)) bad = true;
          for (int j = 0; j < k; ++j)
            if (load_id<IdT>(op.ids, row + j) == id) bad = true;
          m |= 1ull << c.expert_rank[id];
        }
      }
      if (bad) {
        m = 0;
        report_error(c, kInvalidRoute, kPhaseDispatch, 1, static_cast<unsigned>(t));
      }
      mask_arr[t] = m;
    }
    // Position of this token among the tile's rows for each destination: the first eight
    // stay packed in registers (one byte each, < 32), wider fan-outs spill to the plane.
    unsigned long long packed = 0;
    int j = 0;
    for (int d = 0; d < W; ++d) {
      const bool bit = (m >> d) & 1ull;
      const unsigned ballot = __ballot_sync(0xffffffffu, bit);
      if (bit) {
        const unsigned before = __popc(ballot & ((1u << lane) - 1u));
        if (j < 8) packed |= static_cast<unsigned long long>(before) << (8 * j);
        else dest_rows[static_cast<long long>(t) * fan + j] = static_cast<int>(before);
        ++j;
      }
      if (lane == 0) s_warp_cnt[warp][d] = __popc(ballot);
    }
    __syncthreads();
    if (tid < W) {
      int run = 0;
      for (int w = 0; w < kWarps; ++w) {
        const int v = s_warp_cnt[w][tid];
        s_warp_cnt[w][tid] = run;
        run += v;
      }
      tile_cnt[static_cast<long long>(tile) * W + tid] = run;
    }
    __syncthreads();
    if (m) {
      int jj = 0;
      for (unsigned long long mm = m; mm; mm &= mm - 1, ++jj) {
        const int d = __ffsll(static_cast<long long>(mm)) - 1;
        const long long at = static_cast<long long>(t) * fan + jj;
        const int before = jj < 8 ? static_cast<int>((packed >> (8 * jj)) & 0xffu) : dest_rows[at];
        dest_rows[at] = before + s_warp_cnt[warp][d];
      }
    }
    __syncthreads();
  }

  prof.stamp(1);
  if (!solo && !rank_barrier(c, &hdr->bar_count, gridDim.x, kPhaseDispatch)) return;
  prof.stamp(2);
  debug_delay(c, 1);

  // ---- 2. publish my count row ----------------------------------------------
  // One warp per destination: the lanes fetch the tiles' counts together (one memory round
  // trip for 32 tiles instead of one per tile) and scan them with shuffles.
  for (int d = warp; d < W; d += kWarps) {
    int run = 0;
    for (int first = 0; first < ntiles; first += 32) {
      const int tile = first + lane;
      const int v = tile < ntiles ? tile_cnt[static_cast<long long>(tile) * W + d] : 0;
      int upto = v;
#pragma unroll
      for (int step = 1; step < 32; step <<= 1) {
        const int below = __shfl_up_sync(0xffffffffu, upto, step);
        if (lane >= step) upto += below;
      }
      if (tile < ntiles) tile_base[tile * W + d] = run + upto - v;
      run += __shfl_sync(0xffffffffu, upto, 31);
    }
    if (lane == 0) s_send[d] = run;
  }
  __syncthreads();
  if (blockIdx.x == 0 && !lone) {
    for (int i = tid; i < W * W; i += kThreads) {
      const int p = i / W, d = i % W;
      unsigned long long* dst = reinterpret_cast<unsigned long long*>(s_heap[p] + cl.cnt) +
                                (static_cast<size_t>(par) * W + self) * W + d;
      st_relaxed_sys(dst, tagged(g, static_cast<unsigned>(s_send[d])));
    }
  }

  // ---- 4a. payload, first loads --------------------------------------------------------
  // Movers (warps 0..kMovers-1 of every CTA) claim row pieces from the rank's counter. Which
  // rows to read only depends on this rank's routing, so the first batch of loads is issued
  // here and is in flight while the counts of the other ranks are awaited below.
  const long long row_bytes = static_cast<long long>(H) * 2;
  const int pieces = static_cast<int>((row_bytes + kMoveStageBytes - 1) / kMoveStageBytes);
  const int piece_bytes = static_cast<int>(align_up((row_bytes + pieces - 1) / pieces, 16));
  const long long move_items = static_cast<long long>(T) * pieces;
  const bool mover = kVec16 && warp < kMovers;
  char* const ring = reinterpret_cast<char*>(tile_base) + op.ring_offset +
                     static_cast<size_t>(warp < kMovers ? warp : 0) * kMoveStages * kMoveStageBytes;
  unsigned long long* const mfull = s_mfull + (warp < kMovers ? warp : 0) * kMoveStages;
  // Small batches are spread one piece per claim; large ones fill every stage of a mover.
  const long long per_mover = move_items / (static_cast<long long>(gridDim.x) * kMovers);
  const unsigned claim = per_mover < 1 ? 1u : (per_mover > kMoveStages ? kMoveStages : static_cast<unsigned>(per_mover));
  int b_tok[kMoveStages], b_bytes[kMoveStages];
  long long b_b0[kMoveStages];
  unsigned long long b_mask[kMoveStages];
  unsigned mparity = 0;        // bit i: phase parity of stage i's barrier
  bool more = mover;
  // Towards the end of the batch a mover takes one piece at a time: a full claim is tens of
  // microseconds of link time, which the last claimers would spend alone.
  const long long tail_items = static_cast<long long>(gridDim.x) * kMovers * kMoveStages;
  // Every mover's FIRST claim is its own fixed share (mover g of the launch takes pieces
  // g * claim ...): hundreds of movers hitting one counter at the same instant queue up for
  // microseconds. The counter hands out what lies behind those shares.
  const long long fixed_items = static_cast<long long>(gridDim.x) * kMovers * claim;
  bool first_claim = true;
  auto claim_and_load = [&]() {
    unsigned base = 0, taken = claim;
    if (first_claim) {
      base = (blockIdx.x * kMovers + warp) * claim;
      first_claim = false;
    } else if (lane == 0) {
      const long long handed = fixed_items + static_cast<long long>(ld_volatile_u32(&hdr->work_next));
      if (claim > 1 && move_items - handed < tail_items) taken = 1;
      base = static_cast<unsigned>(fixed_items) + atomicAdd(&hdr->work_next, taken);
    }
    base = __shfl_sync(0xffffffffu, base, 0);
    taken = __shfl_sync(0xffffffffu, taken, 0);
#pragma unroll
    for (int i = 0; i < kMoveStages; ++i) {
      const long long item = static_cast<long long>(base) + i;
      b_mask[i] = 0ull;
      if (i < static_cast<int>(taken) && item < move_items) {
        const int t = static_cast<int>(item / pieces);
        const long long b0 = (item - static_cast<long long>(t) * pieces) * piece_bytes;
        b_tok[i] = t;
        b_b0[i] = b0;
        b_bytes[i] = static_cast<int>(min(row_bytes, b0 + piece_bytes) - b0);
        b_mask[i] = mask_arr[t];
        if (b_mask[i] != 0ull && lane == 0) {
          mbarrier_arrive_expect_tx(mfull + i, static_cast<unsigned>(b_bytes[i]));
          bulk_load_to_smem(ring + static_cast<size_t>(i) * kMoveStageBytes,
                            reinterpret_cast<const char*>(op.x) + static_cast<long long>(t) * row_bytes + b0,
                            static_cast<unsigned>(b_bytes[i]), mfull + i);
        }
      }
    }
    more = static_cast<long long>(base) + taken < move_items;
  };
  if (mover) claim_and_load();

  // ---- 3. wait for every rank's counts and addresses ---------------------------
  // A word of a LATER generation in this parity's place means the group is out of step (a rank
  // ran more dispatches than this one): that is reported at once instead of timing out.
  bool ok = true;
  for (int i = tid; i < W * W && ok && !lone; i += kThreads) {
    bool ahead = false;
    ok = bounded_wait(c, kPhaseDispatch, 3, [&] {
      const unsigned tag = tag_of(ld_acquire_sys(my_cnt + i));
      ahead = static_cast<int>(tag - g) > 0;
      return tag == g || ahead;
    }, prof.poll_counter());
    if (ok && ahead) {
      report_error(c, kIdentityMismatch, kPhaseDispatch, 7, static_cast<unsigned>(i / W));
      ok = false;
    }
  }
  for (int i = tid; i < W * 5 && ok && !lone; i += kThreads) {
    const unsigned long long* word = my_addr + (i / 5) * kAddrWords + i % 5;
    ok = bounded_wait(c, kPhaseDispatch, 4, [&] { return tag_of(ld_acquire_sys(word)) == g; }, prof.poll_counter());
  }
  if (!__syncthreads_and(ok)) {
    // Giving up: the loads already issued still target this CTA's shared memory, so they are
    // waited for (bounded) before the CTA may exit.
    if (mover) {
#pragma unroll
      for (int i = 0; i < kMoveStages; ++i)
        if (b_mask[i] != 0ull) mbarrier_wait_bounded(mfull + i, (mparity >> i) & 1u, c.timeout_ns);
    }
    return;
  }
  prof.stamp(3);
  if (tid == 0 && W > 1) prof.first(kProfFirstReceive);
  debug_delay(c, 2);

  if (tid < W) {
    const int d = tid;
    int off = 0, total = 0;
    for (int s = 0; s < W && !lone; ++s) {
      const int v = static_cast<int>(value_of(ld_relaxed_sys(my_cnt + s * W + d)));
      if (s < self) off += v;
      total += v;
    }
    if (lone) total = s_send[0];
    const unsigned long long base = lone ? op.slot_off
        : static_cast<unsigned long long>(value_of(ld_relaxed_sys(my_addr + d * kAddrWords + 0))) << 8;
    const int layout_cap = lone ? op.slot_capacity : static_cast<int>(value_of(ld_relaxed_sys(my_addr + d * kAddrWords + 1)));
    const int bound = lone ? op.capacity : static_cast<int>(value_of(ld_relaxed_sys(my_addr + d * kAddrWords + 2)));
    const unsigned ident = lone ? static_cast<unsigned>(op.identity) : value_of(ld_relaxed_sys(my_addr + d * kAddrWords + 3));
    s_ctas[d] = lone ? static_cast<int>(gridDim.x) : static_cast<int>(value_of(ld_relaxed_sys(my_addr + d * kAddrWords + 4)));
    const SlotLayout pl = slot_layout(layout_cap, 0, H, K, W);
    char* peer_slot = s_heap[d] + base;
    s_planes[d].hidden = peer_slot + pl.hidden;
    s_planes[d].ids = peer_slot + pl.ids;
    s_planes[d].weights = peer_slot + pl.weights;
    s_planes[d].inverse = peer_slot + pl.inverse;
    s_planes[d].ret = peer_slot + pl.ret;
    s_off[d] = off;
    s_total[d] = total;
    s_ok[d] = (total <= bound && bound <= layout_cap) ? 1 : 0;
    if (blockIdx.x == 0) {
      reinterpret_cast<unsigned long long*>(slot + sl.peer_off)[d] = base;
      reinterpret_cast<int*>(slot + sl.peer_cap)[d] = layout_cap;
      reinterpret_cast<int*>(slot + sl.send_cnt)[d] = s_ok[d] ? s_send[d] : 0;
      reinterpret_cast<int*>(slot + sl.recv_cnt)[d] = lone ? s_send[0] : static_cast<int>(value_of(ld_relaxed_sys(my_cnt + d * W + self)));
      if (!s_ok[d] && (d == self || s_send[d] > 0))
        report_error(c, kCapacityExceeded, kPhaseDispatch, static_cast<unsigned>(d), static_cast<unsigned>(total));
      if (ident != static_cast<unsigned>(op.identity))
        report_error(c, kIdentityMismatch, kPhaseDispatch, static_cast<unsigned>(d), ident);
    }
  }
  __syncthreads();

  // ---- 4. payload --------------------------------------------------------------
  if (kVec16) {
    if (mover) {
      // Stores of the batch whose loads are in flight, then the next claim. Lane j issues the
      // copy to the j-th destination; every lane tracks its own copies (bulk async-groups are
      // per thread) and all of them have read the stage before it is refilled.
      bool moving = true;
      while (moving) {
#pragma unroll
        for (int i = 0; i < kMoveStages; ++i) {
          const unsigned long long m = b_mask[i];
          if (m == 0ull || !moving) continue;                       // warp-uniform
          if (!__all_sync(0xffffffffu, mbarrier_wait_bounded(mfull + i, (mparity >> i) & 1u, c.timeout_ns))) {
            if (lane == 0) report_error(c, kTimeout, kPhaseDispatch, 8, static_cast<unsigned>(b_tok[i]));
            moving = false;
            continue;
          }
          mparity ^= 1u << i;
          fence_proxy_async();
          const int t = b_tok[i], n = __popcll(m), tile = t / kRouteTile;
          for (int j = lane; j < n; j += 32) {
            const int d = nth_set_bit(m, j);
            if (!s_ok[d]) continue;
            const long long row = static_cast<long long>(s_off[d]) + tile_base[tile * W + d] +
                                  dest_rows[static_cast<long long>(t) * fan + j];
            bulk_store_from_smem(s_planes[d].hidden + row * row_bytes + b_b0[i],
                                 ring + static_cast<size_t>(i) * kMoveStageBytes, static_cast<unsigned>(b_bytes[i]));
            prof.moved(b_b0[i] == 0 ? 1 : 0, static_cast<unsigned long long>(b_bytes[i]));
          }
        }
        bulk_commit_group();
        bulk_wait_all_read();
        if (!more || !moving) break;
        claim_and_load();
      }
      bulk_wait_all_complete();
      fence_proxy_async();     // the rows went out through the async proxy; the signal below is an ordinary store
    } else {
      // Row metadata: translated local expert ids, weights, inverse entry and return slot of
      // every (token, destination), and this rank's record of where each row went.
      const int meta_warps = kWarps - kMovers;
      const int first = static_cast<int>(blockIdx.x) * meta_warps + (warp - kMovers);
      const int step = static_cast<int>(gridDim.x) * meta_warps;
      for (int t = first; t < T; t += step) {
        const unsigned long long m = mask_arr[t];
        if (m == 0ull) continue;
        const int n = __popcll(m), tile = t / kRouteTile;
        for (int k0 = 0; k0 < K; k0 += 32) {
          const int k = k0 + lane;
          long long local = -1;
          int owner = -1;
          float w = 0.f;
          if (k < K) {
            const long long id = load_id<IdT>(op.ids, static_cast<long long>(t) * K + k);
            if (id >= 0) {
              w = op.weights[static_cast<long long>(t) * K + k];
              owner = c.expert_rank[id];
              local = c.expert_local[id];
            }
          }
          unsigned long long rest = m;
          for (int j = 0; j < n; ++j, rest &= rest - 1) {
            const int d = __ffsll(static_cast<long long>(rest)) - 1;
            if (!s_ok[d]) continue;
            const long long row = static_cast<long long>(s_off[d]) + tile_base[tile * W + d] +
                                  dest_rows[static_cast<long long>(t) * fan + j];
            if (k < K) {
              reinterpret_cast<long long*>(s_planes[d].ids)[row * K + k] = owner == d ? local : -1;
              reinterpret_cast<float*>(s_planes[d].weights)[row * K + k] = w;
            }
            if (k == 0) {
              long long* inv = reinterpret_cast<long long*>(s_planes[d].inverse) + row * 2;
              inv[0] = self;
              inv[1] = t;
              reinterpret_cast<int*>(s_planes[d].ret)[row] = t * fan + j;
            }
          }
        }
        for (int j = lane; j < n; j += 32) {
          const int d = nth_set_bit(m, j);
          send_rows[static_cast<long long>(t) * fan + j] =
              s_ok[d] ? s_off[d] + tile_base[tile * W + d] + dest_rows[static_cast<long long>(t) * fan + j] : -1;
        }
      }
    }
  } else {
  constexpr int kChunk = kVec16 ? 16 : 4;
  constexpr int kUnroll = 4;
  const int segs = op.segments;
  const long long seg_bytes = align_up((row_bytes + segs - 1) / segs, 32 * kChunk);
  const long long items = static_cast<long long>(T) * segs;
  // Work items are claimed from a rank-local counter: SMs differ in how fast their
  // stores drain towards NVLink, and a static split leaves the fast ones idle.
  unsigned next_claim = lane == 0 ? atomicAdd(&hdr->work_next, 1u) : 0u;
  while (true) {
    const long long item = __shfl_sync(0xffffffffu, next_claim, 0);
    if (item >= items) break;
    if (lane == 0) next_claim = atomicAdd(&hdr->work_next, 1u);   // in flight while this item is copied
    const int t = static_cast<int>(item / segs), seg = static_cast<int>(item % segs);
    const unsigned long long m = mask_arr[t];
    if (!m) continue;
    const int n = __popcll(m);
    const int tile = t / kRouteTile;
    for (int j0 = 0; j0 < n; j0 += 32) {   // n <= 63: at most two rounds
      const int j = j0 + lane;
      int d = 0;
      long long row = -1;
      if (j < n) {
        d = nth_set_bit(m, j);
        if (s_ok[d]) row = static_cast<long long>(s_off[d]) + tile_base[tile * W + d] + dest_rows[static_cast<long long>(t) * fan + j];
      }
      // Payload of this round of destinations.
      const int round = min(32, n - j0);
      const long long b0 = seg * seg_bytes;
      const long long b1 = min(row_bytes, b0 + seg_bytes);
      const char* src = reinterpret_cast<const char*>(op.x) + static_cast<long long>(t) * row_bytes;
      for (long long batch = b0; batch < b1; batch += 32ll * kChunk * kUnroll) {   // warp-uniform trip count
        const long long off = batch + static_cast<long long>(lane) * kChunk;
        uint4 v16[kUnroll];
        unsigned v4[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const long long o = off + static_cast<long long>(u) * 32 * kChunk;
          if (o < b1) {
            if (kVec16) v16[u] = *reinterpret_cast<const uint4*>(src + o);
            else v4[u] = *reinterpret_cast<const unsigned*>(src + o);
          }
        }
        for (int jj = 0; jj < round; ++jj) {
          const int d2 = __shfl_sync(0xffffffffu, d, jj);
          const long long r2 = __shfl_sync(0xffffffffu, row, jj);
          if (r2 < 0) continue;
          if (lane == 0 && batch == b0) prof.moved(seg == 0 ? 1 : 0, static_cast<unsigned long long>(b1 - b0));
          char* dst = s_planes[d2].hidden + r2 * row_bytes;
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const long long o = off + static_cast<long long>(u) * 32 * kChunk;
            if (o < b1) {
              if (kVec16) st_payload16(dst + o, v16[u]);
              else st_payload4(dst + o, v4[u]);
            }
          }
        }
      }
      // Row metadata rides with segment 0.
      if (seg == 0) {
        for (int jj = 0; jj < round; ++jj) {
          const int d2 = __shfl_sync(0xffffffffu, d, jj);
          const long long r2 = __shfl_sync(0xffffffffu, row, jj);
          if (r2 < 0) continue;
          long long* out_ids = reinterpret_cast<long long*>(s_planes[d2].ids) + r2 * K;
          float* out_w = reinterpret_cast<float*>(s_planes[d2].weights) + r2 * K;
          for (int k = lane; k < K; k += 32) {
            const long long id = load_id<IdT>(op.ids, static_cast<long long>(t) * K + k);
            long long local = -1;
            float w = 0.f;
            if (id >= 0) {
              w = op.weights[static_cast<long long>(t) * K + k];
              if (c.expert_rank[id] == d2) local = c.expert_local[id];
            }
            out_ids[k] = local;
            out_w[k] = w;
          }
          if (lane == 0) {
            long long* inv = reinterpret_cast<long long*>(s_planes[d2].inverse) + r2 * 2;
            inv[0] = self;
            inv[1] = t;
            reinterpret_cast<int*>(s_planes[d2].ret)[r2] = t * fan + j0 + jj;
          }
        }
        if (j < n) send_rows[static_cast<long long>(t) * fan + j] = static_cast<int>(row);
      }
    }
  }

  }   // register path
  // ---- 5. signal -----------------------------------------------------------------
  const int valid = s_ok[self] ? s_total[self] : 0;
  debug_delay(c, 3);
  __syncthreads();
  prof.stamp(4);
  if (tid < 32) {
    // This CTA's peer stores are performed system-wide before it tells anybody: one fence by the
    // whole first warp (cumulative over the CTA's stores through the barrier above), then lane d
    // counts this CTA in at destination d - every rank that gets rows from this one waits for
    // as many arrivals as this launch has CTAs. (A group of one rank has no peers: device scope
    // is enough there.) No election of a last CTA and no second fence sit on the peers' path.
    if (W > 1) __threadfence_system(); else __threadfence();
    for (int d = tid; d < W; d += 32) {
      if (d == self || !s_ok[d] || s_send[d] <= 0) continue;
      unsigned long long* arrivals = reinterpret_cast<unsigned long long*>(s_heap[d] + cl.done) +
                                     static_cast<size_t>(par) * W + self;
      red_add_relaxed_sys(arrivals, 1ull);
      prof.first(kProfFirstPublish);
    }
    if (tid == 0) {
      const unsigned prev = atomicAdd(&hdr->done_count, 1u);
      s_last = (prev == gridDim.x - 1) ? 1 : 0;
      if (s_last) __threadfence();   // acquire side of the arrival counter
    }
  }
  __syncthreads();
  if (s_last && tid == 0) {          // rank-local bookkeeping of the launch
    misc[kValidCount] = valid;
    misc[kDirtyRows] = valid;
    hdr->bar_count = 0;
    hdr->done_count = 0;
    hdr->work_next = 0;
    hdr->disp_epoch = g;
    __threadfence();
  }

  prof.stamp(5);
  // ---- 6. receive side -------------------------------------------------------------
  // Rows in [valid, previous valid) held data of the slot's previous operation.
  if (dirty_prev > valid) {
    const long long pad_rows = dirty_prev - valid;
    char* hid = slot + sl.hidden;
    long long* ids_out = reinterpret_cast<long long*>(slot + sl.ids);
    float* w_out = reinterpret_cast<float*>(slot + sl.weights);
    long long* inv_out = reinterpret_cast<long long*>(slot + sl.inverse);
    const long long threads = static_cast<long long>(gridDim.x) * kThreads;
    const long long me = static_cast<long long>(blockIdx.x) * kThreads + tid;
    for (long long i = me; i < pad_rows * K; i += threads) {
      ids_out[static_cast<long long>(valid) * K + i] = -1;
      w_out[static_cast<long long>(valid) * K + i] = 0.f;
    }
    for (long long i = me; i < pad_rows * 2; i += threads) inv_out[static_cast<long long>(valid) * 2 + i] = -1;
    if (op.zero_padding) {
      const long long words = pad_rows * row_bytes / 4;
      unsigned* base = reinterpret_cast<unsigned*>(hid + static_cast<long long>(valid) * row_bytes);
      if (kVec16) {
        const long long vecs = words / 4;
        for (long long i = me; i < vecs; i += threads) st_payload16(base + i * 4, make_uint4(0, 0, 0, 0));
      } else {
        for (long long i = me; i < words; i += threads) base[i] = 0u;
      }
    }
  }
  prof.stamp(6);
  ok = true;
  // (Not for this rank's own rows: the launch itself completes only when they are written.)
  // Every CTA of a source counts itself in once its rows for this rank are stored. The counter
  // belongs to this generation's parity and goes back to zero below, for the generation after
  // next (no source can be there before this rank has entered the next generation, i.e.
  // finished this one).
  if (tid < W && tid != self && s_ok[self] && value_of(ld_relaxed_sys(my_cnt + tid * W + self)) > 0) {
    const unsigned long long expected = static_cast<unsigned long long>(s_ctas[tid]);
    ok = bounded_wait(c, kPhaseDispatch, 6, [&] { return ld_acquire_sys(my_done + tid) >= expected; },
                      prof.poll_counter());
  }
  if (__syncthreads_and(ok) && W > 1) {
    // The CTA that is through last puts the counters back (the others no longer read them).
    if (tid == 0) {
      __threadfence();
      s_last = atomicAdd(&hdr->fin_count, 1u) == gridDim.x - 1 ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
      if (tid < W) st_relaxed_sys(my_done + tid, 0ull);
      if (tid == 0) hdr->fin_count = 0;
    }
  }
  prof.stamp(7);
  prof.flush(&hdr->status);
  sample_end(op.samples, sample);
}

template <typename IdT, bool kVec16, bool kProfile>
__global__ void __launch_bounds__(kThreads, 1) dispatch_kernel(const __grid_constant__ DispatchArgs args) {
  extern __shared__ __align__(128) int tile_base[];
  dispatch_body<IdT, kVec16, kProfile>(args.op[blockIdx.y], tile_base);
}

using DispatchKernel = void (*)(const DispatchArgs);

// The profiling specialisations are separate kernels: an ordinary launch carries no timers.
template <bool kProfile>
DispatchKernel pick_kernel_of(bool ids64, bool vec16) {
  if (ids64) return vec16 ? dispatch_kernel<long long, true, kProfile> : dispatch_kernel<long long, false, kProfile>;
  return vec16 ? dispatch_kernel<int, true, kProfile> : dispatch_kernel<int, false, kProfile>;
}
DispatchKernel pick_kernel(bool ids64, bool vec16, bool profile = false) {
  return profile ? pick_kernel_of<true>(ids64, vec16) : pick_kernel_of<false>(ids64, vec16);
}

}  // namespace

size_t dispatch_ring_offset(int max_tokens, int world) {
  return align_up(static_cast<size_t>(route_tiles(max_tokens) + 1) * world * sizeof(int), 128);
}

size_t dispatch_dynamic_smem(int max_tokens, int world, bool vec16) {
  return dispatch_ring_offset(max_tokens, world) + (vec16 ? kMoveRingBytes : 0);
}

cudaError_t dispatch_max_ctas(bool ids64, bool vec16, size_t dynamic_smem, int* ctas) {
  int device = 0, sms = 0, per_sm = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (err != cudaSuccess) return err;
  DispatchKernel kernel = pick_kernel(ids64, vec16);
  if (dynamic_smem > 48 * 1024) {
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(dynamic_smem));
    if (err != cudaSuccess) return err;
  }
  err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, dynamic_smem);
  if (err != cudaSuccess) return err;
  *ctas = per_sm * sms;
  return cudaSuccess;
}

cudaError_t launch_dispatch(const DispatchArgs& args, int ranks, int ctas_per_rank, bool ids64, bool vec16,
                            size_t dynamic_smem, bool cooperative, cudaStream_t stream) {
  DispatchKernel kernel = pick_kernel(ids64, vec16, args.op[0].profile != nullptr);
  if (dynamic_smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(dynamic_smem));
    if (err != cudaSuccess) return err;
  }
  void* params[] = {const_cast<DispatchArgs*>(&args)};
  if (!cooperative)
    return cudaLaunchKernel(reinterpret_cast<const void*>(kernel), dim3(ctas_per_rank, ranks, 1),
                            dim3(kThreads, 1, 1), params, dynamic_smem, stream);
  return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), dim3(ctas_per_rank, ranks, 1),
                                     dim3(kThreads, 1, 1), params, dynamic_smem, stream);
}

}  // namespace epx
