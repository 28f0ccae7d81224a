// Prepared operator and Python bindings of the NVLink transport.
//
// `Engine` plays the role of the reference's PreparedHostSM
// (ep_xpress/csrc/host_sm.h, ep_xpress/csrc/host_sm.cu:2674-3173): placement,
// peer pointer tables and launch geometry are validated and uploaded ONCE;
// each operation only checks its own tensors and enqueues one cooperative
// launch. One engine drives one rank in production, or several ranks that
// share a GPU when a whole group is emulated inside a single launch.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <optional>
#include <sstream>
#include <stdexcept>
#include <vector>

#include "epx_launch.h"
#include "heap.h"
#include "host_helpers.h"

namespace py = pybind11;

namespace epx {
void bind_moe(py::module_& m);        // moe_bindings.cpp
void bind_host_ring(py::module_& m);  // host_ring.cpp
namespace {

void cuda_check(cudaError_t err, const char* what) {
  if (err != cudaSuccess) {
    std::ostringstream message;
    message << "ep_xpress_b200: " << what << ": " << cudaGetErrorString(err);
    throw std::runtime_error(message.str());
  }
}

cudaStream_t stream_of(int64_t handle) { return reinterpret_cast<cudaStream_t>(handle); }

class Engine {
 public:
  Engine(int world, std::vector<int> local_ranks, int hidden, int topk, std::vector<int> expert_to_rank,
         std::vector<std::vector<int64_t>> heaps, double timeout_seconds, bool single_round, int device,
         bool cooperative)
      : world_(world), local_ranks_(std::move(local_ranks)), hidden_(hidden), topk_(topk), device_(device),
        cooperative_(cooperative) {
    TORCH_CHECK(world >= 1 && world <= kMaxWorld, "world size must be in [1, 63]");
    TORCH_CHECK(!local_ranks_.empty() && local_ranks_.size() <= static_cast<size_t>(kMaxEmulatedRanks),
                "an engine drives between 1 and ", kMaxEmulatedRanks, " ranks");
    TORCH_CHECK(heaps.size() == local_ranks_.size(), "one heap table per local rank is required");
    TORCH_CHECK(hidden > 0 && hidden % 2 == 0, "hidden size must be positive and even");
    TORCH_CHECK(topk > 0 && topk <= 256, "topk must be in [1, 256]");
    TORCH_CHECK(!expert_to_rank.empty(), "expert_to_rank must contain at least one expert");
    TORCH_CHECK(timeout_seconds > 0 && timeout_seconds <= 3600, "timeout must be in (0, 3600] seconds");
    c10::cuda::CUDAGuard guard(device_);
    const int experts = static_cast<int>(expert_to_rank.size());
    std::vector<int> local_index(experts), next(world, 0);
    for (int e = 0; e < experts; ++e) {
      TORCH_CHECK(expert_to_rank[e] >= 0 && expert_to_rank[e] < world, "expert owner is outside the group");
      local_index[e] = next[expert_to_rank[e]]++;
    }
    experts_per_rank_ = next;
    cuda_check(cudaMalloc(&tables_, sizeof(int) * experts * 2), "cudaMalloc expert tables");
    cuda_check(cudaMemcpy(tables_, expert_to_rank.data(), sizeof(int) * experts, cudaMemcpyHostToDevice), "upload");
    cuda_check(cudaMemcpy(tables_ + experts, local_index.data(), sizeof(int) * experts, cudaMemcpyHostToDevice),
               "upload");
    std::vector<RankCtx>& host = host_ctx_;
    host.resize(local_ranks_.size());
    for (size_t i = 0; i < local_ranks_.size(); ++i) {
      TORCH_CHECK(local_ranks_[i] >= 0 && local_ranks_[i] < world, "local rank is outside the group");
      TORCH_CHECK(heaps[i].size() == static_cast<size_t>(world), "a heap table needs one address per rank");
      RankCtx& c = host[i];
      std::memset(&c, 0, sizeof(c));
      c.rank = local_ranks_[i];
      c.world = world;
      c.hidden = hidden;
      c.topk = topk;
      c.num_experts = experts;
      c.single_round = single_round ? 1 : 0;
      c.timeout_ns = static_cast<unsigned long long>(timeout_seconds * 1e9);
      c.expert_rank = tables_;
      c.expert_local = tables_ + experts;
      for (int r = 0; r < world; ++r) {
        TORCH_CHECK(heaps[i][r] != 0, "null heap address");
        HeapRegistry::instance().check_range(reinterpret_cast<void*>(heaps[i][r]), ctrl_layout(world).bytes);
        c.heap[r] = reinterpret_cast<char*>(heaps[i][r]);
      }
      own_heap_.push_back(c.heap[c.rank]);
    }
    cuda_check(cudaMalloc(&ctx_, sizeof(RankCtx) * host.size()), "cudaMalloc rank contexts");
    cuda_check(cudaMemcpy(ctx_, host.data(), sizeof(RankCtx) * host.size(), cudaMemcpyHostToDevice), "upload");
    cuda_check(cudaDeviceGetAttribute(&sms_, cudaDevAttrMultiProcessorCount, device_), "query SM count");
    int supported = 0;
    cuda_check(cudaDeviceGetAttribute(&supported, cudaDevAttrCooperativeLaunch, device_), "query cooperative launch");
    TORCH_CHECK(supported || !cooperative_, "the transport kernels need cooperative all-resident launches");
  }

  ~Engine() {
    if (ctx_ != nullptr) cudaFree(ctx_);
    if (tables_ != nullptr) cudaFree(tables_);
  }

  // Debugging: every CTA sleeps a pseudo-random time below `ns` at each phase boundary, which
  // shakes the interleaving of ranks and CTAs without changing any result.
  void set_debug_delay(int64_t ns) {
    TORCH_CHECK(ns >= 0 && ns <= 1000000, "debug delay must be within [0, 1 ms]");
    c10::cuda::CUDAGuard guard(device_);
    for (RankCtx& c : host_ctx_) c.debug_delay_ns = static_cast<unsigned>(ns);
    cuda_check(cudaDeviceSynchronize(), "quiesce before changing the debug delay");
    cuda_check(cudaMemcpy(ctx_, host_ctx_.data(), sizeof(RankCtx) * host_ctx_.size(), cudaMemcpyHostToDevice),
               "upload rank contexts");
  }
  // 0: the sequential combine protocol (push, signal, wait, reduce) everywhere; anything else:
  // the mailbox protocol (push and reduce side by side, one arrival word per row) wherever it
  // applies. Every rank of a group must make the same choice.
  void set_combine_streaming(int mode) { streaming_ = mode; }
  // Whether the mailbox combine protocol applies to this group's shape (16-byte rows, fan-out
  // up to eight, two or more ranks); tensors that are not 16-byte aligned still fall back.
  bool can_mailbox() const { return combine_can_mailbox(hidden_ % 8 == 0, route_fanout(topk_, world_), world_, static_cast<long long>(hidden_) * 2); }
  int sm_count() const { return sms_; }
  std::vector<int> experts_per_rank() const { return experts_per_rank_; }
  size_t ctrl_bytes() const { return ctrl_layout(world_).bytes; }

  py::dict layout(int64_t capacity, int64_t tokens) const {
    const SlotLayout l = slot_layout(capacity, tokens, hidden_, topk_, world_);
    py::dict d;
    d["hidden"] = l.hidden; d["ids"] = l.ids; d["weights"] = l.weights; d["inverse"] = l.inverse;
    d["partial"] = l.partial; d["ret"] = l.ret; d["staging"] = l.staging; d["mask"] = l.mask; d["dest_rows"] = l.dest_rows; d["send_rows"] = l.send_rows; d["tile_cnt"] = l.tile_cnt;
    d["peer_off"] = l.peer_off; d["peer_cap"] = l.peer_cap; d["send_cnt"] = l.send_cnt; d["recv_cnt"] = l.recv_cnt;
    d["misc"] = l.misc; d["output"] = l.output; d["bytes"] = l.bytes;
    return d;
  }

  // Largest per-rank CTA count a cooperative launch of every variant may use.
  int max_ctas(int64_t max_tokens) const {
    c10::cuda::CUDAGuard guard(device_);
    int best = 1 << 30;
    for (int ids64 = 0; ids64 < 2; ++ids64)
      for (int vec = 0; vec < 2; ++vec) {
        int ctas = 0;
        const size_t smem = dispatch_dynamic_smem(static_cast<int>(max_tokens), world_, vec != 0);
        cuda_check(dispatch_max_ctas(ids64, vec, smem, &ctas), "dispatch occupancy query");
        best = std::min(best, ctas);
      }
    for (int vec = 0; vec < 2; ++vec) {
      int ctas = 0;
      cuda_check(combine_max_ctas(vec, route_fanout(topk_, world_), &ctas), "combine occupancy query");
      best = std::min(best, ctas);
    }
    return best / static_cast<int>(local_ranks_.size());
  }

  at::Tensor view(int local, int64_t offset, std::vector<int64_t> shape, py::object dtype) const {
    check_local(local);
    const auto scalar = torch::python::detail::py_object_to_dtype(dtype);
    int64_t count = 1;
    for (int64_t s : shape) count *= s;
    const size_t bytes = static_cast<size_t>(count) * c10::elementSize(scalar);
    HeapRegistry::instance().check_range(own_heap_[local] + offset, bytes == 0 ? 1 : bytes);
    auto options = at::TensorOptions().dtype(scalar).device(at::kCUDA, device_);
    return at::from_blob(own_heap_[local] + offset, shape, options);
  }

  void slot_reset(int local, int64_t offset, int64_t capacity, int64_t tokens, int64_t stream) const {
    check_local(local);
    c10::cuda::CUDAGuard guard(device_);
    const SlotLayout l = slot_layout(capacity, tokens, hidden_, topk_, world_);
    HeapRegistry::instance().check_range(own_heap_[local] + offset, l.bytes);
    cuda_check(launch_slot_reset(own_heap_[local] + offset, l, capacity, hidden_, topk_, stream_of(stream)),
               "slot reset launch");
  }

  void dispatch(const std::vector<at::Tensor>& x, const std::vector<at::Tensor>& ids,
                const std::vector<at::Tensor>& weights, const std::vector<int64_t>& slot_off,
                const std::vector<int64_t>& capacity, const std::vector<int64_t>& slot_capacity,
                const std::vector<int64_t>& slot_tokens, uint64_t identity, int ctas, bool zero_padding,
                int64_t stream, const std::optional<at::Tensor>& profile,
                const std::optional<at::Tensor>& samples) const {
    const size_t n = local_ranks_.size();
    TORCH_CHECK(x.size() == n && ids.size() == n && weights.size() == n && slot_off.size() == n &&
                capacity.size() == n && slot_capacity.size() == n && slot_tokens.size() == n,
                "dispatch needs one entry per local rank");
    c10::cuda::CUDAGuard guard(device_);
    DispatchArgs args;
    std::memset(&args, 0, sizeof(args));
    bool ids64 = false, vec16 = hidden_ % 8 == 0;
    int64_t max_tokens = 1, max_slot_tokens = 1;
    for (size_t i = 0; i < n; ++i) {
      TORCH_CHECK(x[i].is_cuda() && x[i].get_device() == device_ && ids[i].is_cuda() && weights[i].is_cuda(),
                  "dispatch inputs must live on the context device");
      TORCH_CHECK(x[i].scalar_type() == at::kBFloat16 && x[i].dim() == 2 && x[i].size(1) == hidden_ &&
                  x[i].is_contiguous(), "x must be contiguous BF16 [tokens, hidden]");
      const int64_t tokens = x[i].size(0);
      TORCH_CHECK((ids[i].scalar_type() == at::kInt || ids[i].scalar_type() == at::kLong) && ids[i].dim() == 2 &&
                  ids[i].size(0) == tokens && ids[i].size(1) == topk_ && ids[i].is_contiguous(),
                  "topk_ids must be contiguous int32 or int64 [tokens, topk]");
      TORCH_CHECK(weights[i].scalar_type() == at::kFloat && weights[i].dim() == 2 && weights[i].size(0) == tokens &&
                  weights[i].size(1) == topk_ && weights[i].is_contiguous(),
                  "topk_weights must be contiguous FP32 [tokens, topk]");
      TORCH_CHECK(tokens <= slot_tokens[i], "more tokens than the slot was created for");
      TORCH_CHECK(capacity[i] >= 0 && capacity[i] <= slot_capacity[i], "receive capacity exceeds the slot");
      TORCH_CHECK(reinterpret_cast<uintptr_t>(x[i].data_ptr()) % 4 == 0, "x must be 4-byte aligned");
      TORCH_CHECK(slot_off[i] % kSlotAlign == 0, "slot offsets are 256-byte aligned");
      const bool this64 = ids[i].scalar_type() == at::kLong;
      TORCH_CHECK(i == 0 || this64 == ids64, "all ranks of one launch must use the same id dtype");
      ids64 = this64;
      if (reinterpret_cast<uintptr_t>(x[i].data_ptr()) % 16 != 0) vec16 = false;
      max_tokens = std::max<int64_t>(max_tokens, tokens);
      max_slot_tokens = std::max<int64_t>(max_slot_tokens, slot_tokens[i]);
      const SlotLayout l = slot_layout(slot_capacity[i], slot_tokens[i], hidden_, topk_, world_);
      HeapRegistry::instance().check_range(own_heap_[i] + slot_off[i], l.bytes);
      DispatchOp& op = args.op[i];
      op.ctx = ctx_ + i;
      op.x = x[i].data_ptr();
      op.ids = ids[i].data_ptr();
      op.weights = weights[i].data_ptr<float>();
      op.slot_off = static_cast<unsigned long long>(slot_off[i]);
      op.identity = identity & 0xffffffffull;
      op.tokens = static_cast<int>(tokens);
      op.capacity = static_cast<int>(capacity[i]);
      op.slot_capacity = static_cast<int>(slot_capacity[i]);
      op.slot_tokens = static_cast<int>(slot_tokens[i]);
      op.ids64 = this64 ? 1 : 0;
      op.zero_padding = zero_padding ? 1 : 0;
    }
    TORCH_CHECK(route_tiles(static_cast<int>(max_tokens)) <= kMaxRouteTiles, "too many tokens for one dispatch");
    const size_t smem = dispatch_dynamic_smem(static_cast<int>(max_tokens), world_, vec16);
    ctas = std::max(1, ctas);
    const int segments = pick_segments(max_tokens, ctas);
    for (size_t i = 0; i < n; ++i) {
      args.op[i].segments = segments;
      args.op[i].vec16 = vec16 ? 1 : 0;
      args.op[i].ring_offset = static_cast<int>(dispatch_ring_offset(static_cast<int>(max_tokens), world_));
    }
    attach_profile(profile, ctas, n, [&](size_t i, unsigned long long* p) { args.op[i].profile = p; });
    attach_samples(samples, n, [&](size_t i, unsigned long long* ring, int capacity) {
      args.op[i].samples = ring; args.op[i].sample_capacity = capacity;
    });
    cuda_check(launch_dispatch(args, static_cast<int>(n), ctas, ids64, vec16, smem, cooperative_, stream_of(stream)),
               "dispatch launch");
  }

  void combine(const std::vector<std::optional<at::Tensor>>& partial, const std::vector<at::Tensor>& out,
               const std::vector<int64_t>& slot_off, const std::vector<int64_t>& slot_capacity,
               const std::vector<int64_t>& slot_tokens, uint64_t identity, int ctas, int64_t stream,
               const std::optional<at::Tensor>& profile, int mailbox, const std::optional<at::Tensor>& samples) const {
    const size_t n = local_ranks_.size();
    TORCH_CHECK(partial.size() == n && out.size() == n && slot_off.size() == n && slot_capacity.size() == n &&
                slot_tokens.size() == n, "combine needs one entry per local rank");
    c10::cuda::CUDAGuard guard(device_);
    CombineArgs args;
    std::memset(&args, 0, sizeof(args));
    bool vec16 = hidden_ % 8 == 0;
    int64_t max_tokens = 1, max_rows = 1;
    for (size_t i = 0; i < n; ++i) {
      TORCH_CHECK(out[i].is_cuda() && out[i].get_device() == device_ && out[i].scalar_type() == at::kBFloat16 &&
                  out[i].dim() == 2 && out[i].size(1) == hidden_ && out[i].is_contiguous(),
                  "combine output must be contiguous BF16 [tokens, hidden] on the context device");
      TORCH_CHECK(out[i].size(0) <= slot_tokens[i], "more tokens than the slot was created for");
      const SlotLayout l = slot_layout(slot_capacity[i], slot_tokens[i], hidden_, topk_, world_);
      HeapRegistry::instance().check_range(own_heap_[i] + slot_off[i], l.bytes);
      CombineOp& op = args.op[i];
      op.ctx = ctx_ + i;
      op.out = out[i].data_ptr();
      op.slot_off = static_cast<unsigned long long>(slot_off[i]);
      op.identity = identity & 0xffffffffull;
      op.tokens = static_cast<int>(out[i].size(0));
      op.slot_capacity = static_cast<int>(slot_capacity[i]);
      op.slot_tokens = static_cast<int>(slot_tokens[i]);
      if (reinterpret_cast<uintptr_t>(op.out) % 16 != 0) vec16 = false;
      TORCH_CHECK(reinterpret_cast<uintptr_t>(op.out) % 4 == 0, "combine output must be 4-byte aligned");
      TORCH_CHECK(partial[i].has_value(), "combine needs this rank's partial tensor");
      {
        const at::Tensor& p = *partial[i];
        TORCH_CHECK(p.is_cuda() && p.get_device() == device_ && p.scalar_type() == at::kBFloat16 && p.dim() == 2 &&
                    p.size(1) == hidden_ && p.is_contiguous(),
                    "partial must be contiguous BF16 [rows, hidden] on the context device");
        TORCH_CHECK(p.size(0) <= slot_capacity[i], "partial has more rows than the dispatch capacity");
        op.partial = p.data_ptr();
        op.partial_rows = static_cast<int>(p.size(0));
        TORCH_CHECK(reinterpret_cast<uintptr_t>(op.partial) % 4 == 0, "partial must be 4-byte aligned");
        if (reinterpret_cast<uintptr_t>(op.partial) % 16 != 0) vec16 = false;
      }
      max_tokens = std::max<int64_t>(max_tokens, out[i].size(0));
      max_rows = std::max<int64_t>(max_rows, args.op[i].partial_rows);
    }
    (void)max_rows;
    ctas = std::max(1, ctas);
    const int segments = pick_segments(max_tokens, ctas);
    for (size_t i = 0; i < n; ++i) {
      args.op[i].segments = segments;
      args.op[i].vec16 = vec16 ? 1 : 0;
      // Heralds pay off once the pushers run several rounds: more received rows than the push
      // CTAs move in two rounds of fifteen. (Every rank derives the same answer from the slot.)
      args.op[i].herald = slot_capacity[i] > 2 * 15 * 64 ? 1 : 0;
    }
    attach_profile(profile, ctas, n, [&](size_t i, unsigned long long* p) { args.op[i].profile = p; });
    attach_samples(samples, n, [&](size_t i, unsigned long long* ring, int capacity) {
      args.op[i].samples = ring; args.op[i].sample_capacity = capacity;
    });
    const int fanout = route_fanout(topk_, world_);
    cuda_check(launch_combine(args, static_cast<int>(n), ctas, vec16, fanout, world_, hidden_, mailbox < 0 ? streaming_ != 0 : mailbox != 0, cooperative_,
                              stream_of(stream)), "combine launch");
  }

  void scale_rows(const at::Tensor& hidden, const at::Tensor& local_ids, const at::Tensor& weights,
                  const at::Tensor& valid_count, const std::optional<at::Tensor>& factors, at::Tensor& partial,
                  int64_t stream) const {
    c10::cuda::CUDAGuard guard(device_);
    TORCH_CHECK(hidden.is_cuda() && hidden.scalar_type() == at::kBFloat16 && hidden.dim() == 2 &&
                hidden.size(1) == hidden_ && hidden.is_contiguous(), "hidden must be contiguous BF16 [rows, hidden]");
    const int64_t rows = hidden.size(0);
    TORCH_CHECK(local_ids.scalar_type() == at::kLong && local_ids.is_contiguous() && local_ids.size(0) == rows &&
                local_ids.size(1) == topk_, "local_ids must be contiguous int64 [rows, topk]");
    TORCH_CHECK(weights.scalar_type() == at::kFloat && weights.is_contiguous() && weights.size(0) == rows &&
                weights.size(1) == topk_, "weights must be contiguous FP32 [rows, topk]");
    TORCH_CHECK(valid_count.scalar_type() == at::kInt && valid_count.numel() == 1, "valid_count must be int32[1]");
    TORCH_CHECK(partial.scalar_type() == at::kBFloat16 && partial.is_contiguous() && partial.size(0) >= rows &&
                partial.size(1) == hidden_, "partial must be contiguous BF16 [>= rows, hidden]");
    const float* f = nullptr;
    int nf = 0;
    if (factors.has_value()) {
      TORCH_CHECK(factors->scalar_type() == at::kFloat && factors->is_contiguous() && factors->numel() > 0,
                  "factors must be a non-empty contiguous FP32 tensor");
      f = factors->data_ptr<float>();
      nf = static_cast<int>(factors->numel());
    }
    cuda_check(launch_scale_rows(hidden.data_ptr(), local_ids.data_ptr<int64_t>() == nullptr ? nullptr :
                                 reinterpret_cast<const long long*>(local_ids.data_ptr<int64_t>()),
                                 weights.data_ptr<float>(), valid_count.data_ptr<int>(), f, nf, partial.data_ptr(),
                                 static_cast<int>(rows), hidden_, topk_, stream_of(stream)), "scale_rows launch");
  }

  // Synchronises the device and returns (status, detail, dispatch epoch, combine epoch).
  py::tuple status(int local) const {
    check_local(local);
    c10::cuda::CUDAGuard guard(device_);
    CtrlHeader header;
    cuda_check(cudaMemcpy(&header, own_heap_[local], sizeof(header), cudaMemcpyDeviceToHost), "status readback");
    return py::make_tuple(header.status, header.error_detail, header.disp_epoch, header.comb_epoch);
  }

  // Debug window onto the control words of a rank: lets a test play a peer by
  // writing flag words from the CPU (technique of the reference's
  // tests/test_host_sm_native_cuda.py:176-186, which forges words in a mapped arena).
  void poke_u64(int local, int64_t offset, uint64_t value) const {
    check_local(local);
    TORCH_CHECK(offset >= 0 && offset % 8 == 0 && static_cast<size_t>(offset) + 8 <= ctrl_bytes(),
                "offset is outside the control region");
    c10::cuda::CUDAGuard guard(device_);
    cuda_check(cudaMemcpy(own_heap_[local] + offset, &value, 8, cudaMemcpyHostToDevice), "poke");
  }
  uint64_t peek_u64(int local, int64_t offset) const {
    check_local(local);
    TORCH_CHECK(offset >= 0 && offset % 8 == 0 && static_cast<size_t>(offset) + 8 <= ctrl_bytes(),
                "offset is outside the control region");
    c10::cuda::CUDAGuard guard(device_);
    uint64_t value = 0;
    cuda_check(cudaMemcpy(&value, own_heap_[local] + offset, 8, cudaMemcpyDeviceToHost), "peek");
    return value;
  }
  py::dict ctrl_offsets() const {
    const CtrlLayout l = ctrl_layout(world_);
    py::dict d;
    d["cnt"] = l.cnt; d["addr"] = l.addr; d["done"] = l.done; d["ready"] = l.ready; d["ident"] = l.ident;
    d["perr"] = l.perr; d["bytes"] = l.bytes;
    return d;
  }

 private:
  void check_local(int local) const {
    TORCH_CHECK(local >= 0 && static_cast<size_t>(local) < local_ranks_.size(), "local rank index out of range");
  }
  // Rows are split into segments of at least 2 KiB (one fully unrolled warp iteration) so
  // that small batches still occupy every warp. Work items are claimed dynamically, so two
  // items per warp are enough for balance; more would only add per-item overhead.
  int pick_segments(int64_t tokens, int ctas) const {
    const int64_t warps = static_cast<int64_t>(ctas) * (kThreads / 32);
    const int64_t row_bytes = static_cast<int64_t>(hidden_) * 2;
    const int64_t max_segments = std::max<int64_t>(1, row_bytes / 2048);
    const int64_t wanted = (2 * warps + std::max<int64_t>(tokens, 1) - 1) / std::max<int64_t>(tokens, 1);
    return static_cast<int>(std::max<int64_t>(1, std::min(wanted, max_segments)));
  }
  // profile: int64 [ranks, ctas, kProfileStamps] on the context device, or nothing.
  template <typename Assign>
  void attach_profile(const std::optional<at::Tensor>& profile, int ctas, size_t ranks, Assign assign) const {
    if (!profile.has_value()) return;
    const at::Tensor& p = *profile;
    TORCH_CHECK(p.is_cuda() && p.get_device() == device_ && p.scalar_type() == at::kLong && p.is_contiguous() &&
                p.numel() >= static_cast<int64_t>(ranks) * ctas * kProfileStamps,
                "profile must be a contiguous int64 CUDA tensor of at least ranks * ctas * 8 elements");
    for (size_t i = 0; i < ranks; ++i)
      assign(i, reinterpret_cast<unsigned long long*>(p.data_ptr<int64_t>()) + i * ctas * kProfileStamps);
  }

  // samples: int64 [ranks, 1 + capacity, kSampleWords] on the context device, or nothing.
  template <typename Assign>
  void attach_samples(const std::optional<at::Tensor>& samples, size_t ranks, Assign assign) const {
    if (!samples.has_value()) return;
    const at::Tensor& t = *samples;
    TORCH_CHECK(t.is_cuda() && t.get_device() == device_ && t.scalar_type() == at::kLong && t.is_contiguous() &&
                t.dim() == 3 && t.size(0) == static_cast<int64_t>(ranks) && t.size(1) >= 2 && t.size(2) == kSampleWords,
                "samples must be a contiguous int64 CUDA tensor [ranks, 1 + capacity, 4]");
    for (size_t i = 0; i < ranks; ++i)
      assign(i, reinterpret_cast<unsigned long long*>(t.data_ptr<int64_t>()) + i * t.size(1) * kSampleWords,
             static_cast<int>(t.size(1) - 1));
  }

  int world_;
  std::vector<int> local_ranks_;
  int hidden_, topk_, device_;
  bool cooperative_ = true;
  std::vector<RankCtx> host_ctx_;
  int streaming_ = -1;
  int sms_ = 0;
  std::vector<int> experts_per_rank_;
  std::vector<char*> own_heap_;
  int* tables_ = nullptr;
  RankCtx* ctx_ = nullptr;
};

}  // namespace
}  // namespace epx

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  using namespace epx;
  m.doc() = "ep_xpress_b200 native runtime (sm_100a)";
  m.attr("MAX_WORLD") = kMaxWorld;
  m.attr("MAX_EMULATED_RANKS") = kMaxEmulatedRanks;
  m.attr("THREADS") = kThreads;
  m.attr("PROFILE_STAMPS") = kProfileStamps;
  m.attr("SAMPLE_WORDS") = kSampleWords;
  m.def("heap_allocate", [](size_t bytes) { return reinterpret_cast<int64_t>(HeapRegistry::instance().allocate(bytes)); });
  m.def("heap_export", [](int64_t base) { return py::bytes(HeapRegistry::instance().export_handle(reinterpret_cast<void*>(base))); });
  m.def("heap_open", [](const std::string& handle, size_t bytes) {
    return reinterpret_cast<int64_t>(HeapRegistry::instance().open(handle, bytes));
  });
  m.def("heap_release", [](int64_t base) { HeapRegistry::instance().release(reinterpret_cast<void*>(base)); });
  m.def("heap_live_mappings", [] { return HeapRegistry::instance().live_mappings(); });
  m.def("ctrl_bytes", [](int world) { return ctrl_layout(world).bytes; });
  m.def("slot_bytes", [](int64_t capacity, int64_t tokens, int hidden, int topk, int world) {
    return slot_layout(capacity, tokens, hidden, topk, world).bytes;
  });
  // ---- helpers of the host-staged transport (host_helpers.cu) ----
  m.def("register_host", [](int64_t address, size_t bytes) { register_host_range(reinterpret_cast<void*>(address), bytes); });
  m.def("unregister_host", [](int64_t address) { unregister_host_range(reinterpret_cast<void*>(address)); });
  m.def("registered_host_ranges", [] { return registered_host_ranges(); });
  m.def("copy_d2h_async", [](const at::Tensor& source, int64_t host_address, int64_t stream) {
    TORCH_CHECK(source.is_cuda() && source.is_contiguous(), "the source must be a contiguous CUDA tensor");
    c10::cuda::CUDAGuard guard(source.device());
    cuda_check(copy_device_to_registered_host(source.data_ptr(), reinterpret_cast<void*>(host_address),
                                              static_cast<size_t>(source.numel()) * source.element_size(),
                                              stream_of(stream)), "device-to-host copy");
  });
  m.def("add_partial", [](at::Tensor& accum, const at::Tensor& partial, const at::Tensor& index, at::Tensor& status,
                          int64_t stream) {
    TORCH_CHECK(accum.is_cuda() && accum.scalar_type() == at::kFloat && accum.dim() == 2 && accum.is_contiguous(),
                "accum must be a contiguous FP32 CUDA tensor [tokens, hidden]");
    TORCH_CHECK(partial.is_cuda() && partial.scalar_type() == at::kBFloat16 && partial.dim() == 2 &&
                partial.is_contiguous() && partial.size(1) == accum.size(1),
                "partial must be a contiguous BF16 CUDA tensor [rows, hidden]");
    TORCH_CHECK(index.is_cuda() && index.scalar_type() == at::kLong && index.is_contiguous() &&
                index.numel() == partial.size(0), "index must be a contiguous int64 CUDA tensor [rows]");
    TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() == 1, "status must be int32[1]");
    c10::cuda::CUDAGuard guard(accum.device());
    cuda_check(launch_add_partial(accum.data_ptr<float>(), partial.data_ptr(),
                                  reinterpret_cast<const long long*>(index.data_ptr<int64_t>()), partial.size(0),
                                  accum.size(0), static_cast<int>(accum.size(1)), status.data_ptr<int>(),
                                  stream_of(stream)), "add_partial launch");
  });
  m.def("finish_combine", [](const at::Tensor& remote, const at::Tensor& local, at::Tensor& out, bool single_round,
                             int64_t stream) {
    TORCH_CHECK(remote.is_cuda() && remote.scalar_type() == at::kFloat && remote.is_contiguous() &&
                local.is_cuda() && local.scalar_type() == at::kFloat && local.is_contiguous() &&
                local.numel() == remote.numel(), "remote and local must be contiguous FP32 CUDA tensors of one shape");
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.is_contiguous() &&
                out.numel() == remote.numel(), "out must be a contiguous BF16 CUDA tensor of the same shape");
    c10::cuda::CUDAGuard guard(remote.device());
    cuda_check(launch_finish_combine(remote.data_ptr<float>(), local.data_ptr<float>(), out.data_ptr(), remote.numel(),
                                     single_round, stream_of(stream)), "finish_combine launch");
  });
  py::class_<Engine>(m, "Engine")
      .def(py::init<int, std::vector<int>, int, int, std::vector<int>, std::vector<std::vector<int64_t>>, double, bool, int, bool>(),
           py::arg("world"), py::arg("local_ranks"), py::arg("hidden"), py::arg("topk"), py::arg("expert_to_rank"),
           py::arg("heaps"), py::arg("timeout_seconds"), py::arg("single_round"), py::arg("device"),
           py::arg("cooperative") = true)
      .def("sm_count", &Engine::sm_count)
      .def("set_debug_delay", &Engine::set_debug_delay)
      .def("set_combine_streaming", &Engine::set_combine_streaming, py::arg("mode"))
      .def("experts_per_rank", &Engine::experts_per_rank)
      .def("ctrl_bytes", &Engine::ctrl_bytes)
      .def("ctrl_offsets", &Engine::ctrl_offsets)
      .def("layout", &Engine::layout)
      .def("max_ctas", &Engine::max_ctas)
      .def("view", &Engine::view)
      .def("slot_reset", &Engine::slot_reset)
      .def("dispatch", &Engine::dispatch, py::arg("x"), py::arg("ids"), py::arg("weights"), py::arg("slot_off"),
           py::arg("capacity"), py::arg("slot_capacity"), py::arg("slot_tokens"), py::arg("identity"),
           py::arg("ctas"), py::arg("zero_padding"), py::arg("stream"), py::arg("profile") = py::none(),
           py::arg("samples") = py::none())
      .def("combine", &Engine::combine, py::arg("partial"), py::arg("out"), py::arg("slot_off"),
           py::arg("slot_capacity"), py::arg("slot_tokens"), py::arg("identity"), py::arg("ctas"), py::arg("stream"),
           py::arg("profile") = py::none(), py::arg("mailbox") = -1, py::arg("samples") = py::none())
      .def("combine_can_mailbox", &Engine::can_mailbox)
      .def("scale_rows", &Engine::scale_rows)
      .def("status", &Engine::status)
      .def("poke_u64", &Engine::poke_u64)
      .def("peek_u64", &Engine::peek_u64);
  epx::bind_moe(m);
  epx::bind_host_ring(m);
}
