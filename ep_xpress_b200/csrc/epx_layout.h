// Memory layout of one rank's peer-mapped heap, shared by host and device code.
//
// Every rank owns ONE device allocation ("heap") that all peers map over
// NVLink. It starts with a control region (status words, local barrier
// counters and the generation-tagged flag words that peers write) followed by
// operation slots. A slot holds everything one dispatch/combine pair needs:
// the receive tensors that peers store into, the partial-result plane that
// peers load from, and rank-local route state.
//
// The reference keeps the equivalent state in mapped host arenas whose sizes
// are mirrored between Python and the native ABI (ep_xpress/config.py:167-191,
// ep_xpress/csrc/host_sm.cu:2689-2817). Here the wire format is the tensors
// themselves: no frames, no staging copy.
#pragma once
#include <cstddef>
#include <cstdint>

#if defined(__CUDACC__)
#define EPX_HD __host__ __device__ __forceinline__
#else
#define EPX_HD inline
#endif

namespace epx {

constexpr int kMaxWorld = 63;        // destination sets are 64-bit masks
constexpr int kMaxEmulatedRanks = 8; // ranks that one launch may carry on one GPU
constexpr int kThreads = 512;        // threads per CTA of the transport kernels
constexpr int kRouteTile = kThreads; // tokens routed per CTA iteration
constexpr int kSlotAlign = 256;      // every sub-buffer starts on a 256-byte boundary
constexpr int kMaxRouteTiles = 8192; // bound of the per-CTA prefix table
constexpr int kProfileStamps = 24;   // words of one CTA's profile record: 8 phase stamps, then ProfileWord
constexpr int kFlagLine = 128;       // arrival words that follow every staging row (one u32 per row segment)
constexpr int kMaxRowSegments = kFlagLine / 4;

// Sticky status codes (same meaning as ep_xpress/host_sm.py:32-38).
enum Status : int {
  kOk = 0,
  kInvalidRoute = 1,
  kCapacityExceeded = 2,
  kTimeout = 3,
  kPeerAbort = 4,
  kIdentityMismatch = 5,
  kEpochsExhausted = 6,   // 2^31 - 1 operations of one kind ran on this context: re-create it
};
constexpr unsigned kLastEpoch = 0x7ffffffeu;   // generation tags compare as signed differences

EPX_HD size_t align_up(size_t value, size_t alignment) {
  return (value + alignment - 1) / alignment * alignment;
}

// ---- control region -------------------------------------------------------
// Local words live in CtrlHeader. Peer-written words follow it; each is a
// 64-bit (generation << 32 | value) word with exactly one writer.
struct CtrlHeader {
  int status;               // first error code seen by this rank, 0 when healthy
  int abort_flag;           // non-zero once any CTA gave up; others bail out
  unsigned bar_count;       // dispatch grid-barrier arrivals of the running launch
  unsigned done_count;      // dispatch CTAs that finished their stores
  unsigned disp_epoch;      // completed dispatch generations
  unsigned comb_epoch;      // completed combine generations
  unsigned cdone_count;     // combine CTAs whose partial rows are in the heap
  unsigned cfin_count;      // combine CTAs that finished reducing
  unsigned long long error_detail;  // (phase << 56 | where << 32 | value) of the first error
  unsigned work_next;       // dispatch: next unclaimed (token, segment) work item
  unsigned cwork_push;      // combine: next unclaimed (row, segment) item of the push phase
  unsigned cwork_reduce;    // combine: next unclaimed (token, segment) item of the reduce phase
  unsigned fin_count;       // dispatch CTAs that are through with the launch's last wait
  unsigned long long reserved[25];
};
static_assert(sizeof(CtrlHeader) == 256, "control header is one 256-byte block");

constexpr int kAddrWords = 8;         // address words one rank publishes per dispatch

struct CtrlLayout {
  size_t cnt;    // u64 [2][W][W]  counts row of every source, by generation parity
  size_t addr;   // u64 [2][W][8]  (slot offset >> 8, slot capacity, row bound, identity, CTAs of the launch, -, -, -) of every peer
  size_t done;   // u64 [2][W]     CTAs of source s whose rows for this rank are stored (counted up by s, reset by the reader)
  size_t ready;  // u64 [W]        combine: (epoch << 32 | rows of yours I have pushed), monotone, max-updated
  size_t ident;  // u64 [2][W]     diagnostics: operation identity of every peer
  size_t perr;   // u32 [W]        error code published by a failing peer
  size_t hand;   // PushSlot [kMaxPushCtas]  rank-local: rounds that push CTAs hand to herald warps (mailbox combine)
  size_t bytes;  // size of the whole control region
};

// One pusher's hand-over to its herald warp (rank-local: both run in the same launch).
constexpr int kMaxPushCtas = 64;
constexpr int kPushSlotRounds = 4;      // rounds a pusher may run ahead of its herald
constexpr int kPushRoundWords = 16;     // arrival words of one round (one per stage lane; 0 = none)
struct PushSlot {
  unsigned posted;       // rounds whose rows are complete at their owners (release, gpu scope)
  unsigned final_rounds; // 0 while the pusher runs; 1 + its number of rounds once it is done
  unsigned heralded;     // rounds whose arrival words are out
  unsigned reserved[13];
  unsigned long long words[kPushSlotRounds][kPushRoundWords];   // addresses of round r's arrival words at r % kPushSlotRounds
};
static_assert(sizeof(PushSlot) == 64 + 8 * kPushSlotRounds * kPushRoundWords, "hand-over slot layout");

EPX_HD CtrlLayout ctrl_layout(int world) {
  CtrlLayout l;
  const size_t w = static_cast<size_t>(world);
  l.cnt = sizeof(CtrlHeader);
  l.addr = l.cnt + 2 * w * w * 8;
  l.done = l.addr + 2 * w * kAddrWords * 8;
  l.ready = l.done + 2 * w * 8;
  l.ident = l.ready + w * 8;
  l.perr = l.ident + 2 * w * 8;
  l.hand = align_up(l.perr + w * 4, 256);
  l.bytes = align_up(l.hand + sizeof(PushSlot) * kMaxPushCtas, 4096);
  return l;
}

// ---- slot -----------------------------------------------------------------
// The peer-visible part comes first and every plane OFFSET in it depends only on
// (capacity, hidden, topk), so a peer that knows my slot offset and capacity can
// address every plane (the last one, staging, is sized by this rank's token bound,
// but nothing peer-visible follows it). The rank-local part comes after.
struct SlotLayout {
  // peer-visible
  size_t hidden;     // bf16  [capacity, hidden]
  size_t ids;        // int64 [capacity, topk]
  size_t weights;    // f32   [capacity, topk]
  size_t inverse;    // int64 [capacity, 2]
  size_t ret;        // i32   [capacity]           where the row's result goes back: token * fanout + j
  size_t staging;    // [tokens * fanout] x (bf16 [hidden] + kFlagLine bytes of arrival words): partial rows
                     // pushed back by the expert ranks, each followed by the combine epoch per row segment
  // rank-local
  size_t partial;    // bf16  [capacity, hidden]   default output plane of the expert runner
  size_t mask;       // u64   [tokens]             destination-rank set per token
  size_t dest_rows;  // i32   [tokens, fanout]     position among this rank's rows for the j-th destination
  size_t send_rows;  // i32   [tokens, fanout]     final row index at the j-th destination (-1: not sent)
  size_t tile_cnt;   // i32   [tiles, world]       per route tile, rows per destination
  size_t peer_off;   // u64   [world]              slot offset inside each peer's heap
  size_t peer_cap;   // i32   [world]              capacity of each peer's slot
  size_t send_cnt;   // i32   [world]              rows this rank sent to each peer
  size_t recv_cnt;   // i32   [world]              rows each peer sent to this rank
  size_t misc;       // i32   [64]  valid_count, dirty_rows, ...
  size_t output;     // bf16  [tokens, hidden]     combine result (workspaces)
  size_t bytes;
};

// Words 8.. of a CTA's profile record (profiling launches only). Words 0..7 are phase stamps
// on the GPU's global timer (combine: 4..7 hold pipeline cycle counts instead).
enum ProfileWord : int {
  kProfRows = 8,          // rows this CTA stored to destination planes (dispatch) or pushed (combine)
  kProfBytes = 9,         // payload bytes of those rows
  kProfItems = 10,        // combine: (token, row segment) items this CTA's producers issued
  kProfPolls = 11,        // iterations of bounded waits on words that peers write
  kProfFirstPublish = 12, // time of this CTA's first publication to a peer (0: none)
  kProfFirstReceive = 13, // time this CTA first saw data or a word from a peer (0: none)
  kProfStatus = 14,       // the rank's status word when the CTA left
  kProfCompletion = 15,   // index of the last phase stamp the CTA wrote
  kProfMode = 16,         // combine: 1 + protocol (0 register, 1 bulk, 2 mailbox); dispatch: 1 register path, 2 bulk-copy movers
  kProfPushWait = 17,     // combine, mailbox: ns the CTA's pushers spent waiting for their copies (loads landed, stores completed)
  kProfArrivalWait = 18,  // combine, mailbox: ns producer 0 spent waiting for arrival words of peers' rows
  kProfStoreCycles = 19,  // combine, bulk-copy reduce: cycles consumer warp 0 spent converting and storing finished chunks
};

enum MiscWord : int { kValidCount = 0, kDirtyRows = 1, kSendTotal = 2 };

EPX_HD int route_fanout(int topk, int world) { return topk < world ? topk : world; }
EPX_HD int route_tiles(int tokens) { return (tokens + kRouteTile - 1) / kRouteTile; }
// Distance between two staging rows: the BF16 row plus its line of arrival words.
EPX_HD size_t staging_stride(int hidden) { return static_cast<size_t>(hidden) * 2 + kFlagLine; }

EPX_HD SlotLayout slot_layout(long long capacity, long long tokens, int hidden, int topk, int world) {
  SlotLayout l;
  const size_t c = static_cast<size_t>(capacity), t = static_cast<size_t>(tokens);
  const size_t h = static_cast<size_t>(hidden), k = static_cast<size_t>(topk);
  const size_t w = static_cast<size_t>(world);
  size_t at = 0;
  auto take = [&](size_t bytes) { size_t here = at; at = align_up(at + bytes, kSlotAlign); return here; };
  l.hidden = take(c * h * 2);
  l.ids = take(c * k * 8);
  l.weights = take(c * k * 4);
  l.inverse = take(c * 16);
  l.ret = take(c * 4);
  l.staging = take(t * static_cast<size_t>(route_fanout(topk, world)) * staging_stride(hidden));
  l.partial = take(c * h * 2);
  l.mask = take(t * 8);
  l.dest_rows = take(t * static_cast<size_t>(route_fanout(topk, world)) * 4);
  l.send_rows = take(t * static_cast<size_t>(route_fanout(topk, world)) * 4);
  l.tile_cnt = take(static_cast<size_t>(route_tiles(static_cast<int>(tokens)) + 1) * w * 4);
  l.peer_off = take(w * 8);
  l.peer_cap = take(w * 4);
  l.send_cnt = take(w * 4);
  l.recv_cnt = take(w * 4);
  l.misc = take(64 * 4);
  l.output = take(t * h * 2);
  l.bytes = align_up(at, 4096);
  return l;
}

// Constant per-rank state; lives in device memory, one instance per rank that
// this process drives (one in production, several when a single GPU emulates a
// whole group inside one cooperative launch).
struct RankCtx {
  int rank;
  int world;
  int hidden;
  int topk;
  int num_experts;
  int single_round;               // 0: remote-sum -> bf16 -> + local -> bf16; 1: one rounding
  unsigned debug_delay_ns;        // debugging: every CTA sleeps a pseudo-random time below this at phase boundaries
  unsigned long long timeout_ns;  // bound of every device-side wait
  const int* expert_rank;         // [num_experts] owner rank
  const int* expert_local;        // [num_experts] index among the owner's experts
  char* heap[kMaxWorld + 1];      // heap base of every rank as mapped into this process
};

struct DispatchOp {
  const RankCtx* ctx;
  const void* x;          // bf16 [tokens, hidden]
  const void* ids;        // int32|int64 [tokens, topk]
  const float* weights;   // f32 [tokens, topk]
  unsigned long long slot_off;
  unsigned long long identity;  // diagnostics: hash of (phase, tag); 0 when off
  unsigned long long* profile;  // null, or [ctas, kProfileStamps] globaltimer stamps of this launch
  unsigned long long* samples;  // null, or a sample ring (kSampleWords below) that replays keep filling
  int sample_capacity;
  int tokens;
  int capacity;           // row bound of this operation (<= slot_capacity)
  int slot_capacity;      // capacity the slot was laid out for
  int slot_tokens;        // token bound the slot was laid out for
  int ids64;
  int segments;           // pieces a row is split into for the payload phase
  int vec16;              // rows are 16-byte aligned and hidden % 8 == 0
  int zero_padding;       // zero hidden rows in [valid, previous valid)
  int ring_offset;        // dynamic shared memory: where the movers' stage rings start (after the tile prefix table)
};

struct CombineOp {
  const RankCtx* ctx;
  const void* partial;    // bf16 [rows, hidden]: this rank's weighted expert output (any device tensor)
  void* out;              // bf16 [tokens, hidden]
  unsigned long long slot_off;
  unsigned long long identity;
  unsigned long long* profile;  // null, or [ctas, kProfileStamps] globaltimer stamps of this launch
  unsigned long long* samples;  // null, or a sample ring (kSampleWords below) that replays keep filling
  int sample_capacity;
  int tokens;
  int slot_capacity;
  int slot_tokens;
  int segments;
  int vec16;
  int partial_rows;       // rows of `partial`; fewer than the received rows is an error
  int herald;             // mailbox protocol: non-zero = arrival words are published by herald CTAs (large batches)
};

// Bounded timing record of operations that run from CUDA graphs (every replay is a new
// operation, the storage is fixed at capture): u64 [1 + capacity][kSampleWords]. Row 0 is the
// header {operations that found the ring full, generation that maps to sample 0, enabled, -},
// written by the host at quiescent points only; row 1 + i belongs to the operation whose
// generation is base + i and holds {earliest CTA start, latest CTA end, CTAs that finished, -}
// on the GPU's global timer (ns). The host presets starts to ~0 and ends to 0.
constexpr int kSampleWords = 4;

struct DispatchArgs { DispatchOp op[kMaxEmulatedRanks]; };
struct CombineArgs { CombineOp op[kMaxEmulatedRanks]; };

}  // namespace epx
