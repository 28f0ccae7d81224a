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
// launches (host_sm.cu:559-590, :1212-1468, :592-607) and, like its mailbox kernel
// (host_sm.cu:1952-2511), receives and reduces in the same kernel. Default protocol
// ("mailbox", groups of two or more ranks, 16-byte rows, fan-out up to eight):
//   push     some CTAs of the launch only push: their pusher warp claims received rows whose
//            token lives on a peer, fifteen per round. A row travels partial -> shared
//            memory -> the owner's staging row as bulk asynchronous copies (TMA, no tensor
//            map); when the copies of a round have completed, the pusher stores the
//            combine epoch into the arrival word that sits right behind each staging row
//            (one system-scope fence per round). No CTA-wide fence, no counter, no "all
//            rows are out" message.
//   reduce   at the same time the other CTAs walk the rank's own tokens:
//            a producer warp polls the arrival words of exactly the rows a token is
//            owed (local memory), copies them into a shared-memory stage, and four
//            consumer warps add them in rank order and store the result.
// The sequential protocol (push everything, fence, one progress word per peer, wait,
// reduce) is kept for rows that are not 16-byte aligned, wider fan-outs, and as a
// selectable fallback. A group of one rank only reduces.
// No trailing handshake is needed: a staging row is only rewritten by the combine
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

// Accumulators hold two FP32 sums per 64-bit register (the two elements of one BF16 pair).
template <int kWords>
__device__ __forceinline__ void accumulate(unsigned long long* acc, const Chunk<kWords>& c) {
#pragma unroll
  for (int i = 0; i < kWords; ++i) acc[i] = add_f32x2(acc[i], bf16x2_to_f32x2(c.w[i]));
}

// Two-step rounding (default) or single rounding of the accumulated sum.
template <int kWords>
__device__ __forceinline__ Chunk<kWords> finish(const unsigned long long* acc, const Chunk<kWords>& local,
                                                bool has_local, bool single_round) {
  Chunk<kWords> out;
#pragma unroll
  for (int i = 0; i < kWords; ++i) {
    unsigned long long sum = acc[i];
    float lo, hi;
    if (!single_round) {
      unpack_f32x2(sum, lo, hi);
      const unsigned long long rounded = bf16x2_to_f32x2(pack_bf16x2(lo, hi));
      sum = add_f32x2(rounded, has_local ? bf16x2_to_f32x2(local.w[i]) : 0ull);
    }
    unpack_f32x2(sum, lo, hi);
    out.w[i] = pack_bf16x2(lo, hi);
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
        unsigned long long acc[kWords];
#pragma unroll
        for (int i = 0; i < kWords; ++i) acc[i] = 0ull;
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
    unsigned long long acc[kWords];
#pragma unroll
    for (int i = 0; i < kWords; ++i) acc[i] = 0ull;
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

// ---- reduce phase, bulk-copy variant -------------------------------------------------------
// (rows 16-byte aligned, at most kPeerBatch contributors per token)
// The reducing warps of a CTA form independent pipelines. Each has two producer warps, four
// consumer warps and a private ring of shared-memory stages. The producers walk the pipeline's
// share of the CTA's (token, row segment) items alternately; lane j issues ONE bulk copy (TMA) of contributor j's
// segment into the stage and all copies of an item complete on the stage's "full" mbarrier.
// The consumers add the staged chunks in ascending rank order, store the result and release
// the stage through its "empty" mbarrier. Data in flight lives in shared memory, so the phase
// needs few registers; a producer's per-item bookkeeping is a serial instruction stream of
// about a microsecond, which is why there are several of them. Route look-ups (mask, row
// indices) are loaded for 32 items at once and one batch ahead.
constexpr int kGroupWarps = 4;                    // consumer warps of one pipeline
constexpr int kGroupThreads = kGroupWarps * 32;
constexpr int kMaxGroups = 4;
constexpr int kGroupProducers = 2;                // producer warps of one pipeline: they take its items alternately
constexpr int kBulkThreads = kThreads + 32 * kMaxGroups * kGroupProducers;   // 4 pipelines of 4 + 2 warps = 24 warps
constexpr size_t kBulkSmemBytes = 192 * 1024;              // ... sharing 192 KB of stage rings
constexpr int kMaxGroupStages = 3;
constexpr int kChunksPerThread = 4;
constexpr int kSegMaxBytes = 16384;               // largest row segment of one item

// Mailbox protocol: the CTAs of a launch split into PUSH CTAs and REDUCE CTAs. A push CTA runs
// one pusher warp that owns the whole shared memory as fifteen row stages; a reduce CTA runs
// four reduce pipelines. The roles live on different SMs because they disturb each other on one:
// every bulk copy of an SM goes through that SM's one copy engine, where the reducers' loads
// queue behind peer stores that the saturated link drains slowly (measured: 3.8 us per reduce
// item next to a pusher, 1.1 us alone), and the system-scope fence in front of a round's
// arrival words waits for every store the SM has in flight.
//
// That fence is the price of a release at system scope: it does not complete while its SM has
// peer stores in flight and holds up the SM's next stores meanwhile (measured at 2 GPUs, 4096
// tokens: pushers done after 113 us with a fence per round, 92 us without). Large batches
// therefore hand every completed round to a HERALD warp on an SM that stores nothing else - a
// few CTAs of the launch hold one herald warp per pusher - which runs the fence and stores the
// arrival words while the pusher already moves its next round. (A herald warp inside the push
// CTA or inside a reduce CTA does not help: the fence stalls whichever SM runs it, and a busy
// SM's fence is as slow as the pusher's own.) Small batches, one round per pusher, keep the
// fence in the pusher: the hand-over would only add latency.
constexpr int kMailGroups = kMaxGroups;
constexpr int kMailThreads = kBulkThreads;
constexpr size_t kMailReduceSmem = kBulkSmemBytes;
constexpr int kPushStages = 15;                   // bulk copies a pusher keeps in flight
constexpr int kPushStageBytes = 14336;
constexpr size_t kMailSmemBytes = static_cast<size_t>(kPushStages) * kPushStageBytes;   // >= kMailReduceSmem
static_assert(kMailSmemBytes >= kMailReduceSmem, "a reduce CTA's rings must fit the launch's shared memory");

// Push CTAs of a mailbox launch of `ctas` CTAs (at least two): enough SMs to keep the link
// busy - a pusher moves fifteen rows per round trip - and the rest reduce, which is the heavier
// job in bytes (every pushed row is read again, plus the local rows and the output). With
// heralds, one CTA per sixteen pushers is taken from the reducers.
__host__ __device__ __forceinline__ int mailbox_push_ctas(int ctas) {
  const int wanted = ctas * 7 / 16;
  return wanted < 1 ? 1 : (wanted > kMaxPushCtas ? kMaxPushCtas : wanted);
}
constexpr int kHeraldWarpsPerCta = 16;
__host__ __device__ __forceinline__ int mailbox_herald_ctas(int push_ctas) {
  return (push_ctas + kHeraldWarpsPerCta - 1) / kHeraldWarpsPerCta;
}
// Smallest launch that has a push CTA, its herald CTA and a reduce CTA.
constexpr int kMinHeraldLaunch = 3;

// Segment size: as large as possible while every group still gets three stages of `fan`
// contributor slots (an item's latency chain - arrival check, copy, reduce, hand-back - is
// several times its reduce time, so two stages leave the consumers waiting); two stages when
// three would push the segments below 2 KiB.
__device__ __forceinline__ int ring_segment_bytes(int fan, size_t group_smem) {
  int fit = static_cast<int>(group_smem / (3 * static_cast<size_t>(fan))) / 512 * 512;
  if (fit < 2048) fit = static_cast<int>(group_smem / (2 * static_cast<size_t>(fan))) / 512 * 512;
  return fit < kSegMaxBytes ? fit : kSegMaxBytes;
}
__device__ __forceinline__ int ring_stages(int fan, int segment_bytes, size_t group_smem) {
  const int fit = static_cast<int>(group_smem / (static_cast<size_t>(fan) * segment_bytes));
  return fit < kMaxGroupStages ? fit : kMaxGroupStages;
}

struct StageItem {
  long long out_offset;   // byte offset of the segment inside the output tensor
  int bytes;              // segment length, multiple of 16
  int contributors;       // n
  int self_index;         // position of this rank among the contributors, or -1
  unsigned valid;         // bit j: contributor j was copied
  int end;                // non-zero: no more items
  int pad;
};

__device__ __forceinline__ void mbarrier_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_address(bar)) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Shared -> global copy of `bytes` (a multiple of 16, both addresses 16-byte aligned) by the
// copy engine of this SM; the destination may be a peer's memory. Completion is tracked by the
// issuing thread's bulk async-groups (commit / wait below). One copy per call, no fan-out.
__device__ __forceinline__ void bulk_store_from_smem(void* dst, const void* src, unsigned bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_address(src)),
               "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Every bulk copy this thread committed has read its source AND its writes are complete.
__device__ __forceinline__ void bulk_wait_all_complete() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

struct BulkReduceArgs {
  const unsigned long long* mask_arr;
  const int* send_rows;
  const char* partial;
  const char* staging;
  char* out;
  long long row_bytes;
  long long stride;       // distance between two staging rows
  int tokens;
  int fan;
  int self;
  int partial_rows;
  bool single_round;
  unsigned long long timeout_ns;
  unsigned long long* profile;
  int cta, ctas;          // this CTA's index among the CTAs that reduce, and their number
  // mailbox launches only
  const RankCtx* ctx;
  unsigned epoch;
};

// Barriers and item slots are indexed [group][stage]. Returns false when a bounded wait gave up.
// Called by the first kGroups * (kGroupWarps + kGroupProducers) warps of the CTA: consumers first,
// then the producer warps, kGroupProducers per group. The producers of a group take its items
// alternately (item k fills stage k % stages whoever issues it), because a producer's per-item
// chain - arrival words, look-ups, barrier, copies - is longer than the consumers' arithmetic. kMailbox: the peers are still pushing while this runs, so before a
// producer copies a token's rows, lane j waits (bounded) for the arrival word behind the staging
// row of remote contributor j to carry this combine's epoch, and the CTAs take items round-robin
// so that each of them owns tokens from every part of the batch.
template <int kGroups, bool kMailbox, size_t kReduceSmem, bool kProfile>
__device__ __forceinline__ bool bulk_reduce(const BulkReduceArgs& a, char* smem, unsigned long long* full_all,
                                            unsigned long long* empty_all, StageItem* items_all,
                                            Profiler<kProfile>& prof) {
  constexpr int kConsumerWarps = kGroups * kGroupWarps;
  constexpr size_t kGroupSmemBytes = kReduceSmem / kGroups;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool producer = warp >= kConsumerWarps;
  const int group = producer ? (warp - kConsumerWarps) / kGroupProducers : warp / kGroupWarps;
  const int turn = producer ? (warp - kConsumerWarps) % kGroupProducers : 0;   // which items of the pipeline this producer takes
  const int seg_max = ring_segment_bytes(a.fan, kGroupSmemBytes);
  const int rsegs = static_cast<int>((a.row_bytes + seg_max - 1) / seg_max);
  const int rseg_bytes = static_cast<int>(align_up((a.row_bytes + rsegs - 1) / rsegs, 512));
  const int items = a.tokens * rsegs;
  const int stages = ring_stages(a.fan, seg_max, kGroupSmemBytes);
  // A wait on a stage's "empty" barrier tells two consecutive phases apart, no more. A producer
  // that takes every kGroupProducers-th item passed the wait of its previous item, i.e. knows
  // that the consumers are at most `stages` + kGroupProducers - 1 items behind: that is within
  // one phase of every stage as long as the ring has at least kGroupProducers stages. A shorter
  // ring (not reachable with the segment sizes above) is filled by the first producer alone.
  const int producers = stages >= kGroupProducers ? kGroupProducers : 1;
  const size_t stage_bytes = static_cast<size_t>(a.fan) * seg_max;
  char* const ring = smem + static_cast<size_t>(group) * kGroupSmemBytes;
  unsigned long long* const full = full_all + group * kMaxGroupStages;
  unsigned long long* const empty = empty_all + group * kMaxGroupStages;
  StageItem* const slots = items_all + group * kMaxGroupStages;
  // Items of this CTA are a contiguous range (local memory only: a static split is balanced),
  // or every ctas-th item in mailbox launches; the groups take them round-robin.
  const int lo = kMailbox ? a.cta : static_cast<int>(static_cast<long long>(items) * a.cta / a.ctas);
  const int hi = static_cast<int>(static_cast<long long>(items) * (a.cta + 1) / a.ctas);
  const int stride = kMailbox ? a.ctas : 1;
  const int cta_items = kMailbox ? (items > lo ? (items - lo + stride - 1) / stride : 0)
                                 : hi - static_cast<int>(static_cast<long long>(items) * a.cta / a.ctas);
  const int mine = cta_items > group ? (cta_items - group + kGroups - 1) / kGroups : 0;
  long long waited = 0, worked = 0, stored = 0;   // profiling only: cycles spent waiting / working / in the store loop
  bool ok = true;
  if (producer) {
    auto item_of = [&](int k) { return lo + (group + k * kGroups) * stride; };
    // Lane L loads the mask of item L of the batch, lane 8q + j the row of contributor j of
    // item 4r + q.
    auto load_batch = [&](int base, unsigned long long& mask, int (&rows)[8]) {
      mask = base + lane < mine ? a.mask_arr[item_of(base + lane) / rsegs] : 0ull;
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int k = base + 4 * r + (lane >> 3), j = lane & 7;
        rows[r] = (k < mine && j < a.fan) ? a.send_rows[static_cast<long long>(item_of(k) / rsegs) * a.fan + j] : -1;
      }
    };
    unsigned long long mask_now = 0, mask_next = 0;
    int rows_now[8], rows_next[8];
    load_batch(0, mask_now, rows_now);
    unsigned use = 0;
    for (int base = 0; base < mine && ok; base += 32) {
      if (base + 32 < mine) load_batch(base + 32, mask_next, rows_next);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        // Mailbox: one look at the arrival words of the next four items (lane 8q + j: contributor
        // j of item 4r + q), so that the words' latency is paid once per four items. A word that
        // already carries the epoch is final; the others are polled again when their item is up.
        unsigned early = a.epoch;
        if (kMailbox) {
          const unsigned long long mk = __shfl_sync(0xffffffffu, mask_now, 4 * r + (lane >> 3));
          const int k = base + 4 * r + (lane >> 3), j = lane & 7;
          if (k < mine && k % producers == turn && j < __popcll(mk) && rows_now[r] >= 0 &&
              nth_set_bit(mk, j) != a.self) {
            const long long tk = item_of(k) / rsegs;
            early = ld_acquire_sys_u32(reinterpret_cast<const unsigned*>(a.staging + (tk * a.fan + j) * a.stride + a.row_bytes));
          }
          __syncwarp();        // the lane that copies a row is not the lane that looked at its word
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int i = 4 * r + q;
          const unsigned long long m = __shfl_sync(0xffffffffu, mask_now, i);
          const int row = __shfl_sync(0xffffffffu, rows_now[r], q * 8 + (lane & 7));
          const unsigned seen = __shfl_sync(0xffffffffu, early, q * 8 + (lane & 7));
          if (base + i >= mine || !ok) continue;                 // warp-uniform
          if ((base + i) % producers != turn) continue;          // the pipeline's other producer fills that stage
          use = static_cast<unsigned>(base + i);                 // stages are used in item order
          const int stage = use % stages;
          const unsigned parity = ((use / stages) & 1u) ^ 1u;
          const long long t0 = clock64();
          if (!__all_sync(0xffffffffu, mbarrier_wait_bounded(empty + stage, parity, a.timeout_ns))) {
            ok = false;
            continue;
          }
          if (kProfile) {
            const long long t1 = clock64();
            waited += t1 - t0;
            worked -= t1 - t0;         // `worked` below adds the whole item: leave the wait out of it
          }
          const int item = item_of(base + i);
          const int t = item / rsegs, seg = item - t * rsegs;
          const int n = __popcll(m);
          const int b0 = seg * rseg_bytes;
          const int bytes = static_cast<int>(min(a.row_bytes, static_cast<long long>(b0) + rseg_bytes)) - b0;
          const char* src = nullptr;
          bool is_self = false;
          if (lane < n) {
            const int d = nth_set_bit(m, lane);
            is_self = d == a.self;
            if (row >= 0 && !(is_self && row >= a.partial_rows))
              src = is_self ? a.partial + static_cast<long long>(row) * a.row_bytes
                            : a.staging + (static_cast<long long>(t) * a.fan + lane) * a.stride;
          }
          if (kMailbox) {
            // Contributor `lane` is a peer: its row is in once the word behind it carries this epoch.
            const bool remote = src != nullptr && !is_self;
            bool fine = true;
            const unsigned long long wait_begin = prof.on() && group == 0 && lane == 0 ? global_timer_ns() : 0ull;
            if (remote && seen != a.epoch) {
              const unsigned* word = reinterpret_cast<const unsigned*>(src + a.row_bytes);
              if (ld_acquire_sys_u32(word) != a.epoch)
                fine = bounded_wait(*a.ctx, kPhaseCombine, 5, [&] { return ld_acquire_sys_u32(word) == a.epoch; },
                                    prof.poll_counter());
            }
            if (remote && fine) prof.first(kProfFirstReceive);
            if (!__all_sync(0xffffffffu, fine)) {
              ok = false;
              continue;
            }
            if (wait_begin != 0ull) prof.count(kProfArrivalWait, global_timer_ns() - wait_begin);
            fence_proxy_async();      // the rows were written by a peer; the copies below read them through the async proxy
          }
          const unsigned valid = __ballot_sync(0xffffffffu, src != nullptr);
          const unsigned self_vote = __ballot_sync(0xffffffffu, is_self);
          if (lane == 0) {
            StageItem& slot = slots[stage];
            slot.out_offset = static_cast<long long>(t) * a.row_bytes + b0;
            slot.bytes = bytes;
            slot.contributors = n;
            slot.self_index = self_vote ? __ffs(self_vote) - 1 : -1;
            slot.valid = valid;
            slot.end = 0;
            prof.count(kProfItems, 1);
            mbarrier_arrive_expect_tx(full + stage, static_cast<unsigned>(__popc(valid)) * static_cast<unsigned>(bytes));
          }
          __syncwarp();
          if (src != nullptr)
            bulk_load_to_smem(ring + static_cast<size_t>(stage) * stage_bytes + lane * seg_max, src + b0,
                              static_cast<unsigned>(bytes), full + stage);
          if (kProfile) worked += clock64() - t0;
        }
      }
      mask_now = mask_next;
#pragma unroll
      for (int r = 0; r < 8; ++r) rows_now[r] = rows_next[r];
    }
    use = static_cast<unsigned>(mine);
    if (ok && mine % producers == turn) {                  // end marker, by the producer whose turn it would be
      const int stage = use % stages;
      const unsigned parity = ((use / stages) & 1u) ^ 1u;
      if (__all_sync(0xffffffffu, mbarrier_wait_bounded(empty + stage, parity, a.timeout_ns))) {
        if (lane == 0) {
          slots[stage].end = 1;
          mbarrier_arrive(full + stage);
        }
      } else {
        ok = false;
      }
    }
  } else {
    // ---------------- consumers: four warps per group, several chunks per thread -------------
    const int gtid = tid % kGroupThreads;
    for (unsigned use = 0;; ++use) {
      const int stage = use % stages;
      const unsigned parity = (use / stages) & 1u;
      const long long t0 = clock64();
      if (!mbarrier_wait_bounded(full + stage, parity, a.timeout_ns)) { ok = false; break; }
      const long long t1 = clock64();
      waited += t1 - t0;
      const StageItem item = slots[stage];
      if (item.end) break;
      const char* base = ring + static_cast<size_t>(stage) * stage_bytes;
      const int chunks = item.bytes / 16;
      for (int first = gtid; first < chunks; first += kGroupThreads * kChunksPerThread) {
        unsigned long long acc[kChunksPerThread][4];
        Chunk<4> local[kChunksPerThread];
#pragma unroll
        for (int u = 0; u < kChunksPerThread; ++u) {
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[u][i] = 0ull;
        }
        bool has_local = false;
        for (int j = 0; j < item.contributors; ++j) {
          if (!((item.valid >> j) & 1u)) continue;
          const bool is_local = !a.single_round && j == item.self_index;
          has_local |= is_local;
#pragma unroll
          for (int u = 0; u < kChunksPerThread; ++u) {
            const int chunk = first + u * kGroupThreads;
            if (chunk < chunks) {
              const uint4 v = *reinterpret_cast<const uint4*>(base + j * seg_max + chunk * 16);
              Chunk<4> c;
              c.w[0] = v.x; c.w[1] = v.y; c.w[2] = v.z; c.w[3] = v.w;
              if (is_local) local[u] = c;
              else accumulate<4>(acc[u], c);
            }
          }
        }
        const long long t2 = kProfile ? clock64() : 0;
#pragma unroll
        for (int u = 0; u < kChunksPerThread; ++u) {
          const int chunk = first + u * kGroupThreads;
          if (chunk < chunks)
            store_chunk<4>(a.out + item.out_offset + chunk * 16, finish<4>(acc[u], local[u], has_local, a.single_round));
        }
        if (kProfile) stored += clock64() - t2;
      }
      __syncwarp();
      if (lane == 0) mbarrier_arrive(empty + stage);
      worked += clock64() - t1;
    }
  }
  if (kProfile && a.profile != nullptr && lane == 0 && (warp == 0 || warp == kConsumerWarps)) {   // group 0 (its first producer)
    unsigned long long* slot = a.profile + static_cast<size_t>(blockIdx.x) * kProfileStamps + (warp == 0 ? 4 : 6);
    slot[0] = static_cast<unsigned long long>(waited);
    slot[1] = static_cast<unsigned long long>(worked);
    if (warp == 0) a.profile[static_cast<size_t>(blockIdx.x) * kProfileStamps + kProfStoreCycles] = static_cast<unsigned long long>(stored);
  }
  return ok;
}

// ---- push phase -----------------------------------------------------------------------------
// Received rows are grouped by source rank. Pushing them in storage order would make every
// rank write to rank 0 first, then rank 1, ... (incast: one ingress port saturated, the rest
// idle). Work items (row, row segment) therefore interleave the peers in blocks of kPushBlock
// rows, starting with the rank after this one, so that at any moment each rank spreads its
// stores over all peers and each peer receives from all ranks.
constexpr int kPushBlock = 8;

struct PushArgs {
  const int* rows_from;     // [W] rows received from each rank
  const int* first_row;     // [W] first row of each rank in the receive buffer
  char* const* stage;       // [W] staging plane of each rank
  const char* partial;
  const int* ret;
  long long row_bytes;
  long long stride;         // distance between two staging rows
  long long seg_bytes;
  int segs;
  int most;                 // most rows received from one peer
  int valid;
  int self;
  int world;
};

// Resolves push item `q` (segments already divided out) to the received row it stands for and
// the rank that owns its token; false when the item is a hole of the interleaved order.
__device__ __forceinline__ bool push_target(const PushArgs& p, long long q, long long* row, int* source) {
  const int peers = p.world - 1;
  const int in_block = static_cast<int>(q % kPushBlock);
  const long long q2 = q / kPushBlock;
  *source = (p.self + 1 + static_cast<int>(q2 % peers)) % p.world;
  const long long from_source = (q2 / peers) * kPushBlock + in_block;
  if (from_source >= p.rows_from[*source]) return false;
  *row = p.first_row[*source] + from_source;
  return *row < p.valid;
}

template <int kWords, int kUnroll, bool kProfile>
__device__ __forceinline__ void push_item(const PushArgs& p, long long item, int lane, Profiler<kProfile>& prof) {
  constexpr int kChunk = kWords * 4;
  const int seg = static_cast<int>(item % p.segs);
  long long row;
  int source;
  if (!push_target(p, item / p.segs, &row, &source)) return;
  const long long back = p.ret[row];
  const char* src = p.partial + row * p.row_bytes;
  char* dst = p.stage[source] + back * p.stride;
  const long long b0 = seg * p.seg_bytes;
  const long long b1 = min(p.row_bytes, b0 + p.seg_bytes);
  if (lane == 0 && b1 > b0) prof.moved(seg == 0 ? 1 : 0, static_cast<unsigned long long>(b1 - b0));
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

// ---- mailbox push ---------------------------------------------------------------------------
// Run by the pusher warp of a push CTA; lane i < kPushStages owns stage i. Per round the
// warp claims one piece per lane with a single atomic (a row of up to kPushStageBytes is one
// piece; towards the end of the batch the rounds shrink to an even share of what is left),
// every lane resolves its piece, loads it into its stage, stores it to the owner's
// staging row and waits for its own copies to complete; then ONE system-scope fence orders the
// round's completed rows before the arrival words, which the lanes that moved a row's last
// piece store relaxed (a release per word would serialise a round trip to the peer per word).
// The copies run in the SM's copy engine; the lanes only issue and wait, in lockstep, so a
// round costs one chain of latencies (claim, look-up, load, store + acknowledgement, fence)
// whatever the number of rows in it.
__device__ __forceinline__ void st_release_gpu_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// `hand`: null = this warp fences and publishes its own arrival words; otherwise completed rounds
// are posted there for the pusher's herald warp.
template <bool kProfile>
__device__ __forceinline__ bool mailbox_push(const PushArgs& p, const RankCtx& c, CtrlHeader* hdr, char* stages,
                                             unsigned long long* full, unsigned epoch, PushSlot* hand, int lane,
                                             int push_ctas, Profiler<kProfile>& prof) {
  const int peers = p.world - 1;
  const long long blocks = (p.most + kPushBlock - 1) / kPushBlock;
  const int pieces = static_cast<int>((p.row_bytes + kPushStageBytes - 1) / kPushStageBytes);
  const int piece_bytes = static_cast<int>(align_up((p.row_bytes + pieces - 1) / pieces, 16));
  const long long items = blocks * peers * kPushBlock * pieces;
  // All pieces of a row travel in the same round, so that the row's arrival word can follow it.
  const unsigned per_round = static_cast<unsigned>(kPushStages / pieces * pieces);
  char* const stage = stages + static_cast<size_t>(lane < kPushStages ? lane : 0) * kPushStageBytes;
  unsigned long long* const bar = full + (lane < kPushStages ? lane : 0);
  unsigned parity = 0;                                  // of this lane's barrier
  unsigned round = 0;
  bool ok = true;
  while (true) {
    unsigned base = 0, take = per_round;
    if (lane == 0) {
      const long long left = items - static_cast<long long>(ld_volatile_u32(&hdr->cwork_push));
      const long long share = ((left > 0 ? left : 0) / pieces + push_ctas - 1) / push_ctas * pieces;
      if (share < static_cast<long long>(take)) take = static_cast<unsigned>(share < pieces ? pieces : share);
      base = atomicAdd(&hdr->cwork_push, take);
    }
    base = __shfl_sync(0xffffffffu, base, 0);
    take = __shfl_sync(0xffffffffu, take, 0);
    if (static_cast<long long>(base) >= items) break;
    const long long item = static_cast<long long>(base) + lane;
    char* dst = nullptr;
    unsigned* word = nullptr;
    int bytes = 0;
    if (lane < static_cast<int>(take) && item < items) {
      const int piece = static_cast<int>(item % pieces);
      long long row;
      int source;
      if (push_target(p, item / pieces, &row, &source)) {
        const long long b0 = static_cast<long long>(piece) * piece_bytes;
        bytes = static_cast<int>(min(p.row_bytes, b0 + piece_bytes) - b0);
        char* dst_row = p.stage[source] + static_cast<long long>(p.ret[row]) * p.stride;
        dst = dst_row + b0;
        if (piece == pieces - 1) word = reinterpret_cast<unsigned*>(dst_row + p.row_bytes);
        mbarrier_arrive_expect_tx(bar, static_cast<unsigned>(bytes));
        bulk_load_to_smem(stage, p.partial + row * p.row_bytes + b0, static_cast<unsigned>(bytes), bar);
      }
    }
    const unsigned long long wait_begin = prof.on() && lane == 0 ? global_timer_ns() : 0ull;
    if (dst != nullptr) {
      if (mbarrier_wait_bounded(bar, parity, c.timeout_ns)) {
        parity ^= 1u;
        fence_proxy_async();
        bulk_store_from_smem(dst, stage, static_cast<unsigned>(bytes));
        prof.moved(word != nullptr ? 1 : 0, static_cast<unsigned long long>(bytes));
      } else {
        ok = false;
      }
    }
    bulk_commit_group();
    bulk_wait_all_complete();
    if (wait_begin != 0ull) prof.count(kProfPushWait, global_timer_ns() - wait_begin);
    fence_proxy_async();               // the copies wrote through the async proxy; the words below are ordinary stores
    if (!__all_sync(0xffffffffu, ok)) break;
    // A round that only met holes of the interleaved order completed no row: nothing to order,
    // nothing to publish (all pieces of a row travel in one round).
    if (!__any_sync(0xffffffffu, word != nullptr)) continue;
    if (hand == nullptr) {
      __threadfence_system();
      if (word != nullptr) {
        st_relaxed_sys_u32(word, epoch);
        prof.first(kProfFirstPublish);
      }
      continue;
    }
    // The round's rows are complete at their owners: its arrival words go to the herald warp,
    // which publishes them behind a system-scope fence while this warp already moves the next
    // round. The pusher runs at most kPushSlotRounds rounds ahead of its herald.
    if (lane == 0 && round >= kPushSlotRounds)
      ok = bounded_wait(c, kPhaseCombine, 9, [&] {
        return ld_acquire_gpu_u32(&hand->heralded) + kPushSlotRounds > round; }, prof.poll_counter());
    if (!__all_sync(0xffffffffu, ok)) break;
    if (lane < kPushRoundWords)
      hand->words[round % kPushSlotRounds][lane] = reinterpret_cast<unsigned long long>(word);
    __syncwarp();
    if (lane == 0) st_release_gpu_u32(&hand->posted, round + 1);
    ++round;
  }
  const bool fine = __all_sync(0xffffffffu, ok);
  if (hand != nullptr && lane == 0) st_release_gpu_u32(&hand->final_rounds, round + 1);
  return fine;
}

// The herald warp of ONE pusher, on an SM whose only stores are arrival words. Whenever the
// pusher has posted rounds: ONE system-scope fence - cumulative over the pusher's completed
// copies, which reached this warp through the release/acquire on `posted` - then the rounds'
// arrival words as relaxed stores (lane l: the word of stage l). A release per word would
// serialise a round trip to the peer per word.
template <bool kProfile>
__device__ __forceinline__ bool mailbox_herald(const RankCtx& c, PushSlot* slot, unsigned epoch, int lane,
                                               Profiler<kProfile>& prof) {
  unsigned done = 0;                                      // rounds whose words are out
  const unsigned long long start = global_timer_ns();
  unsigned spins = 0;
  while (true) {
    unsigned long long both = 0;
    // (posted, final_rounds) in one load; a pusher that is done posts nothing more.
    if (lane == 0) both = ld_acquire_gpu_u64(reinterpret_cast<const unsigned long long*>(&slot->posted));
    both = __shfl_sync(0xffffffffu, both, 0);
    const unsigned posted = static_cast<unsigned>(both), final_rounds = static_cast<unsigned>(both >> 32);
    if (posted == done) {
      if (final_rounds != 0 && done + 1 == final_rounds) return true;
      if ((++spins & 63u) == 0) {
        if (ld_volatile_i32(&header_of(c.heap[c.rank])->abort_flag) != 0) return false;
        if (global_timer_ns() - start > c.timeout_ns) return false;
      }
      continue;
    }
    __threadfence_system();
    for (unsigned round = done; round != posted; ++round) {
      unsigned long long word = 0;
      if (lane < kPushRoundWords) word = ld_relaxed_sys(&slot->words[round % kPushSlotRounds][lane]);
      if (word != 0ull) {
        st_relaxed_sys_u32(reinterpret_cast<unsigned*>(word), epoch);
        prof.first(kProfFirstPublish);
      }
    }
    __syncwarp();
    done = posted;
    if (lane == 0) st_release_gpu_u32(&slot->heralded, done);
  }
}

enum CombineMode : int { kModeRegister = 0, kModeBulk = 1, kModeMailbox = 2 };

template <bool kVec16, int kMode, bool kProfile>
__device__ __forceinline__ void combine_body(const CombineOp& op, char* dynamic_smem) {
  static_assert(kVec16 || kMode == kModeRegister, "the bulk-copy paths need 16-byte rows");
  constexpr bool kBulk = kMode != kModeRegister;
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
  const int* const ret = reinterpret_cast<const int*>(slot + sl.ret);
  const int* const misc = reinterpret_cast<const int*>(slot + sl.misc);
  const char* const partial = reinterpret_cast<const char*>(op.partial);
  const char* const staging = slot + sl.staging;
  const int fan = route_fanout(K, W);
  const long long row_bytes = static_cast<long long>(H) * 2;
  const long long stride = static_cast<long long>(staging_stride(H));

  __shared__ char* s_stage[64];
  __shared__ int s_need[64];
  __shared__ int s_rows_from[64], s_first_row[64];
  __shared__ int s_most;
  __shared__ int s_last;
  __shared__ unsigned long long s_full[kMaxGroups * kMaxGroupStages], s_empty[kMaxGroups * kMaxGroupStages];
  __shared__ unsigned long long s_push_full[kPushStages + 1];
  __shared__ StageItem s_items[kMaxGroups * kMaxGroupStages];

  Profiler<kProfile> prof(op.profile);
  prof.stamp(0);
  if (prof.on() && threadIdx.x == 0) prof.record[kProfMode] = 1 + kMode;
  const unsigned e = ld_volatile_u32(&hdr->comb_epoch) + 1;
  if (e > kLastEpoch) {       // epochs never wrap; uniform over the rank's CTAs
    if (threadIdx.x == 0 && blockIdx.x == 0) report_error(c, kEpochsExhausted, kPhaseCombine, 0xE0, e);
    return;
  }
  const unsigned sample = sample_begin(op.samples, e, op.sample_capacity);
  // Progress words of the sequential protocol carry (epoch << 32 | rows pushed); "everything"
  // is the largest row count.
  const unsigned long long all_pushed = (static_cast<unsigned long long>(e) << 32) | 0xffffffffull;
  if (tid < W) {
    const unsigned long long off = reinterpret_cast<const unsigned long long*>(slot + sl.peer_off)[tid];
    const int cap = reinterpret_cast<const int*>(slot + sl.peer_cap)[tid];
    const SlotLayout pl = slot_layout(cap, 0, H, K, W);
    s_stage[tid] = c.heap[tid] + off + pl.staging;
    s_need[tid] = (tid != self && reinterpret_cast<const int*>(slot + sl.send_cnt)[tid] > 0) ? 1 : 0;
  }
  if (tid == 64) {
    int at = 0, most = 0;
    for (int r = 0; r < W; ++r) {
      const int count = reinterpret_cast<const int*>(slot + sl.recv_cnt)[r];
      s_first_row[r] = at;
      s_rows_from[r] = count;
      at += count;
      if (r != self && count > most) most = count;
    }
    s_most = most;
  }
  if (kBulk) {
    if (tid < kMaxGroups * kMaxGroupStages) {
      mbarrier_init(s_full + tid, 1);
      mbarrier_init(s_empty + tid, kGroupWarps);
    }
    if (tid >= 96 && tid < 96 + kPushStages) mbarrier_init(s_push_full + (tid - 96), 1);

    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  // Every received row owes its owner a partial row: a shorter `partial` cannot be combined.
  // The rows that exist are still pushed; the owners of the others end with a peer-abort status.
  if (misc[kValidCount] > op.partial_rows && tid == 0 && blockIdx.x == 0)
    report_error(c, kCapacityExceeded, kPhaseCombine, 7, static_cast<unsigned>(op.partial_rows));
  const int valid = min(misc[kValidCount], op.partial_rows);
  const int segs = op.segments;
  const long long seg_bytes = align_up((row_bytes + segs - 1) / segs, 32 * kChunk * kUnroll);
  __syncthreads();

  PushArgs push;
  push.rows_from = s_rows_from; push.first_row = s_first_row; push.stage = s_stage;
  push.partial = partial; push.ret = ret; push.row_bytes = row_bytes; push.stride = stride; push.seg_bytes = seg_bytes;
  push.segs = segs; push.most = s_most; push.valid = valid; push.self = self; push.world = W;
  BulkReduceArgs reduce;
  reduce.mask_arr = mask_arr; reduce.send_rows = send_rows; reduce.partial = partial; reduce.staging = staging;
  reduce.out = reinterpret_cast<char*>(op.out); reduce.row_bytes = row_bytes; reduce.stride = stride;
  reduce.tokens = T; reduce.fan = fan; reduce.self = self; reduce.partial_rows = op.partial_rows;
  reduce.single_round = single_round; reduce.timeout_ns = c.timeout_ns; reduce.profile = op.profile;
  reduce.ctx = &c;
  reduce.epoch = e;

  reduce.cta = static_cast<int>(blockIdx.x);
  reduce.ctas = static_cast<int>(gridDim.x);
  if (kMode == kModeMailbox) {
    // ---- push CTAs, herald CTAs and reduce CTAs side by side ----
    // (A mailbox launch has at least two CTAs; heralds are used from kMinHeraldLaunch CTAs on.)
    const int push_ctas = mailbox_push_ctas(static_cast<int>(gridDim.x));
    const bool heralds = op.herald != 0 && static_cast<int>(gridDim.x) >= kMinHeraldLaunch + 1;
    const int herald_ctas = heralds ? mailbox_herald_ctas(push_ctas) : 0;
    PushSlot* const hand = reinterpret_cast<PushSlot*>(my_heap + cl.hand);
    const int cta = static_cast<int>(blockIdx.x);
    debug_delay(c, 4);
    if (cta < push_ctas) {
      if (tid < 32) {
        if (!mailbox_push<kProfile>(push, c, hdr, dynamic_smem, s_push_full, e, heralds ? hand + cta : nullptr, lane,
                                    push_ctas, prof) && lane == 0)
          report_error(c, kTimeout, kPhaseCombine, 6, 0);
        if (kProfile && prof.on() && lane == 0) prof.record[1] = global_timer_ns();
      }
    } else if (cta < push_ctas + herald_ctas) {
      const int pusher = (cta - push_ctas) * kHeraldWarpsPerCta + (tid >> 5);
      if ((tid >> 5) < kHeraldWarpsPerCta && pusher < push_ctas &&
          !mailbox_herald<kProfile>(c, hand + pusher, e, lane, prof) && lane == 0)
        report_error(c, kTimeout, kPhaseCombine, 8, 0);
    } else {
      reduce.cta = cta - push_ctas - herald_ctas;
      reduce.ctas = static_cast<int>(gridDim.x) - push_ctas - herald_ctas;
      if (!bulk_reduce<kMailGroups, true, kMailReduceSmem, kProfile>(reduce, dynamic_smem, s_full, s_empty, s_items, prof))
        report_error(c, kTimeout, kPhaseCombine, 4, 0);
    }
  } else {
  // ---- A. push my rows to the ranks that own the tokens ---------------------------
  debug_delay(c, 4);
  if (W > 1) {
    const int peers = W - 1;
    const long long blocks = (s_most + kPushBlock - 1) / kPushBlock;
    const long long items = peers > 0 ? blocks * peers * kPushBlock * segs : 0;
    unsigned next_claim = lane == 0 ? atomicAdd(&hdr->cwork_push, 1u) : 0u;
    while (true) {
      const long long item = __shfl_sync(0xffffffffu, next_claim, 0);
      if (item >= items) break;
      if (lane == 0) next_claim = atomicAdd(&hdr->cwork_push, 1u);   // in flight while this item is copied
      push_item<kWords, kUnroll, kProfile>(push, item, lane, prof);
    }
  }
  __syncthreads();
  prof.stamp(1);
  debug_delay(c, 5);

  // A group of one rank has nobody to signal or to wait for.
  if (W > 1) {
    // ---- B. signal ------------------------------------------------------------------------
    if (tid == 0) {
      __threadfence_system();   // this CTA's peer stores are performed system-wide before it arrives
      const unsigned prev = atomicAdd(&hdr->cdone_count, 1u);
      s_last = (prev == gridDim.x - 1) ? 1 : 0;
      if (s_last) __threadfence();   // acquire side of the arrival counter; the update below releases at sys scope
    }
    __syncthreads();
    if (s_last && tid < W && tid != self) {
      unsigned long long* word = reinterpret_cast<unsigned long long*>(c.heap[tid] + cl.ready) + self;
      red_max_release_sys(word, all_pushed);
      prof.first(kProfFirstPublish);
    }

    // ---- C. wait for the peers that push to me ----------------------------------------------
    bool ok = true;
    if (tid < W && s_need[tid]) {
      const unsigned long long* word = reinterpret_cast<const unsigned long long*>(my_heap + cl.ready) + tid;
      ok = bounded_wait(c, kPhaseCombine, 2, [&] { return ld_acquire_sys(word) >= all_pushed; }, prof.poll_counter());
      if (ok) prof.first(kProfFirstReceive);
    }
    if (!__syncthreads_and(ok)) return;
  }
  prof.stamp(2);
  debug_delay(c, 6);

  // ---- D. rank-order reduce from local memory -----------------------------------------------
  if (kBulk) {
    fence_proxy_async();      // the rows were written by generic stores; the reduce reads them through the async proxy
    if (!bulk_reduce<kMaxGroups, false, kBulkSmemBytes, kProfile>(reduce, dynamic_smem, s_full, s_empty, s_items, prof))
      report_error(c, kTimeout, kPhaseCombine, 4, 0);
  } else {
    const long long items = static_cast<long long>(T) * segs;
    while (true) {
      unsigned claimed = 0;
      if (lane == 0) claimed = atomicAdd(&hdr->cwork_reduce, 1u);
      const long long item = __shfl_sync(0xffffffffu, claimed, 0);
      if (item >= items) break;
      if (lane == 0) prof.count(kProfItems, 1);
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
                            : staging + (static_cast<long long>(t) * fan + lane) * stride;
        }
        const unsigned vote_a = __ballot_sync(0xffffffffu, is_self);
        is_self = false;
        if (lane + 32 < n) {
          const int d = nth_set_bit(m, lane + 32);
          const int row = send_rows[static_cast<long long>(t) * fan + lane + 32];
          is_self = (d == self);
          if (row >= 0 && !(is_self && row >= op.partial_rows))
            ptr_b = is_self ? partial + static_cast<long long>(row) * row_bytes
                            : staging + (static_cast<long long>(t) * fan + lane + 32) * stride;
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

      if (n <= kPeerBatch) {
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
  }

  }   // sequential protocol

  // ---- E. retire the epoch ---------------------------------------------------------------
  __syncthreads();
  if (kMode == kModeMailbox) prof.stamp(2);
  prof.stamp(3);
  prof.flush(&hdr->status);
  sample_end(op.samples, sample);
  if (tid == 0) {
    const unsigned prev = atomicAdd(&hdr->cfin_count, 1u);
    if (prev == gridDim.x - 1) {
      hdr->cdone_count = 0;
      hdr->cfin_count = 0;
      hdr->cwork_push = 0;
      hdr->cwork_reduce = 0;
      if (kMode == kModeMailbox && op.herald != 0) {
        PushSlot* hand = reinterpret_cast<PushSlot*>(my_heap + cl.hand);
        for (int i = 0; i < kMaxPushCtas; ++i) { hand[i].posted = 0; hand[i].final_rounds = 0; hand[i].heralded = 0; }
      }
      hdr->comb_epoch = e;
      __threadfence();
    }
  }
}

template <bool kVec16, int kMode, bool kProfile>
__global__ void __launch_bounds__(kMode == kModeMailbox ? kMailThreads : (kMode == kModeBulk ? kBulkThreads : kThreads), 1)
combine_kernel(const __grid_constant__ CombineArgs args) {
  extern __shared__ __align__(128) char combine_smem[];
  combine_body<kVec16, kMode, kProfile>(args.op[blockIdx.y], combine_smem);
}

// ---- a group of ONE rank ----------------------------------------------------------------------
// Nothing is pushed, signalled or awaited: every token's only contributor is this rank's own
// partial row, so combine is one pass over local memory, `out[t] = finish(partial[row(t)])` with
// the same rounding helpers as the general reduce (0 + x in FP32, so -0 becomes +0 there too).
// A pass like that is bound by memory latency, not by arithmetic: it wants many resident warps
// with several 16-byte loads in flight each, not one 640-thread CTA per SM with its stage rings.
// So it is a plain launch of small CTAs, one warp per token at a time. Epoch, sample ring and
// error reporting are those of the general kernel; profiled operations use the general kernel.
constexpr int kLoneThreads = 256;
constexpr int kLoneUnroll = 8;
constexpr int kLoneSms = 148;
constexpr int kLoneMaxCtas = kLoneSms * 8;

__global__ void __launch_bounds__(kLoneThreads) combine_lone_kernel(const __grid_constant__ CombineArgs args) {
  const CombineOp& op = args.op[blockIdx.y];
  const RankCtx& c = *op.ctx;
  const int H = c.hidden, K = c.topk;
  const bool single_round = c.single_round != 0;
  const int tid = threadIdx.x, lane = tid & 31;
  char* const my_heap = c.heap[c.rank];
  CtrlHeader* const hdr = header_of(my_heap);
  const SlotLayout sl = slot_layout(op.slot_capacity, op.slot_tokens, H, K, 1);
  char* const slot = my_heap + op.slot_off;
  const unsigned long long* const mask_arr = reinterpret_cast<const unsigned long long*>(slot + sl.mask);
  const int* const send_rows = reinterpret_cast<const int*>(slot + sl.send_rows);
  const int* const misc = reinterpret_cast<const int*>(slot + sl.misc);
  const char* const partial = reinterpret_cast<const char*>(op.partial);
  char* const out = reinterpret_cast<char*>(op.out);
  const int fan = route_fanout(K, 1);
  const long long row_bytes = static_cast<long long>(H) * 2;

  const unsigned e = ld_volatile_u32(&hdr->comb_epoch) + 1;
  if (e > kLastEpoch) {
    if (tid == 0 && blockIdx.x == 0) report_error(c, kEpochsExhausted, kPhaseCombine, 0xE0, e);
    return;
  }
  const unsigned sample = sample_begin(op.samples, e, op.sample_capacity);
  if (misc[kValidCount] > op.partial_rows && tid == 0 && blockIdx.x == 0)
    report_error(c, kCapacityExceeded, kPhaseCombine, 7, static_cast<unsigned>(op.partial_rows));

  const int warps = kLoneThreads / 32;
  // Warp w of CTA c takes tokens w * grid + c, ...: every CTA (hence every SM) ends up with the
  // same number of rows to within one, also when the grid was rounded up to whole waves.
  for (long long t = static_cast<long long>(tid >> 5) * gridDim.x + blockIdx.x; t < op.tokens;
       t += static_cast<long long>(gridDim.x) * warps) {
    const int row = (mask_arr[t] & 1ull) ? send_rows[t * fan] : -1;
    const bool usable = row >= 0 && row < op.partial_rows;       // warp-uniform
    const char* src = partial + static_cast<long long>(usable ? row : 0) * row_bytes;
    char* dst = out + t * row_bytes;
    for (long long base = static_cast<long long>(lane) * 16; base < row_bytes; base += 32ll * 16 * kLoneUnroll) {
      Chunk<4> v[kLoneUnroll] = {};
#pragma unroll
      for (int u = 0; u < kLoneUnroll; ++u) {
        const long long off = base + static_cast<long long>(u) * 512;
        if (usable && off < row_bytes) v[u] = load_local_chunk<4>(src + off);
      }
#pragma unroll
      for (int u = 0; u < kLoneUnroll; ++u) {
        const long long off = base + static_cast<long long>(u) * 512;
        if (off >= row_bytes) continue;
        unsigned long long acc[4] = {0ull, 0ull, 0ull, 0ull};
        Chunk<4> result;
        if (!usable) {
          result = finish<4>(acc, v[u], false, single_round);          // no contributor: zeros
        } else if (single_round) {
          accumulate<4>(acc, v[u]);
          result = finish<4>(acc, v[u], false, true);
        } else {
          result = finish<4>(acc, v[u], true, false);
        }
        store_chunk<4>(dst + off, result);
      }
    }
  }

  __syncthreads();
  sample_end(op.samples, sample);
  if (tid == 0) {
    __threadfence();
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

struct CombineVariant {
  const void* kernel;
  int threads;
  size_t dynamic_smem;
};

// The bulk-copy reduce needs 16-byte rows and at most kPeerBatch contributors per token; the
// mailbox protocol exists for the bulk-copy reduce and for groups of two or more ranks. The
// profiling specialisations are separate kernels: an ordinary launch carries no timers.
template <bool kProfile>
cudaError_t pick_combine_of(bool vec16, int fanout, bool mailbox, CombineVariant* out) {
  if (vec16 && fanout <= kPeerBatch) {
    if (mailbox) {
      *out = {reinterpret_cast<const void*>(combine_kernel<true, kModeMailbox, kProfile>), kMailThreads, kMailSmemBytes};
      return cudaFuncSetAttribute(combine_kernel<true, kModeMailbox, kProfile>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kMailSmemBytes));
    }
    *out = {reinterpret_cast<const void*>(combine_kernel<true, kModeBulk, kProfile>), kBulkThreads, kBulkSmemBytes};
    return cudaFuncSetAttribute(combine_kernel<true, kModeBulk, kProfile>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(kBulkSmemBytes));
  }
  if (vec16) *out = {reinterpret_cast<const void*>(combine_kernel<true, kModeRegister, kProfile>), kThreads, 0};
  else *out = {reinterpret_cast<const void*>(combine_kernel<false, kModeRegister, kProfile>), kThreads, 0};
  return cudaSuccess;
}
cudaError_t pick_combine(bool vec16, int fanout, bool mailbox, CombineVariant* out, bool profile = false) {
  return profile ? pick_combine_of<true>(vec16, fanout, mailbox, out) : pick_combine_of<false>(vec16, fanout, mailbox, out);
}

}  // namespace

cudaError_t combine_max_ctas(bool vec16, int fanout, int* ctas) {
  int device = 0, sms = 0, per_sm = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (err != cudaSuccess) return err;
  int fewest = 1 << 30;
  for (int mailbox = 0; mailbox < 2; ++mailbox) {
    CombineVariant variant;
    err = pick_combine(vec16, fanout, mailbox != 0, &variant);
    if (err != cudaSuccess) return err;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, variant.kernel, variant.threads, variant.dynamic_smem);
    if (err != cudaSuccess) return err;
    if (per_sm < fewest) fewest = per_sm;
  }
  *ctas = fewest * sms;
  return cudaSuccess;
}

bool combine_can_mailbox(bool vec16, int fanout, int world, long long row_bytes) {
  // (A row travels as at most kPushStages pieces inside one round of a pusher.)
  return vec16 && fanout <= kPeerBatch && world > 1 && row_bytes <= static_cast<long long>(kPushStages) * kPushStageBytes;
}

cudaError_t launch_combine(const CombineArgs& args, int ranks, int ctas_per_rank, bool vec16, int fanout, int world,
                           int hidden, bool mailbox, bool cooperative, cudaStream_t stream) {
  void* params[] = {const_cast<CombineArgs*>(&args)};
  CombineVariant variant;
  const long long row_bytes = static_cast<long long>(hidden) * 2;
  if (world == 1 && ranks == 1 && vec16 && args.op[0].profile == nullptr) {
    // One rank: a streaming pass over local memory, one token per warp and pass.
    const int warps = kLoneThreads / 32, tokens = args.op[0].tokens;
    int ctas = (tokens + warps - 1) / warps;
    if (ctas < 1) ctas = 1;
    if (ctas > kLoneSms) ctas = (ctas + kLoneSms - 1) / kLoneSms * kLoneSms;   // whole waves over the SMs
    if (ctas > kLoneMaxCtas) ctas = kLoneMaxCtas;
    return cudaLaunchKernel(reinterpret_cast<const void*>(combine_lone_kernel), dim3(ctas, 1, 1),
                            dim3(kLoneThreads, 1, 1), params, 0, stream);
  }
  cudaError_t err = pick_combine(vec16, fanout, mailbox && combine_can_mailbox(vec16, fanout, world, row_bytes), &variant,
                                 args.op[0].profile != nullptr);
  if (err != cudaSuccess) return err;
  if (variant.threads == kMailThreads && variant.dynamic_smem == kMailSmemBytes && ctas_per_rank < 2)
    ctas_per_rank = 2;                      // one CTA pushes, one reduces
  const dim3 grid(ctas_per_rank, ranks, 1), block(variant.threads, 1, 1);
  if (!cooperative) return cudaLaunchKernel(variant.kernel, grid, block, params, variant.dynamic_smem, stream);
  return cudaLaunchCooperativeKernel(variant.kernel, grid, block, params, variant.dynamic_smem, stream);
}

}  // namespace epx
