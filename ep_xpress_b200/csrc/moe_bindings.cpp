// Python bindings of the grouped SwiGLU expert runner.
// (Python face of the expert runner; counterpart of fused_experts_valid_count,
// ep_xpress/adapters/sglang_valid.py:233-255.)
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <optional>

#include "moe_gemm.h"

namespace py = pybind11;

namespace epx {
namespace {

void check(cudaError_t err, const char* what) {
  TORCH_CHECK(err == cudaSuccess, "ep_xpress_b200 moe: ", what, ": ", cudaGetErrorString(err));
}

void expect(const at::Tensor& t, at::ScalarType type, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == type, name,
              " must be a contiguous CUDA tensor of the documented dtype");
}

// One forward of the expert runner on `stream`; every buffer is caller-owned.
void moe_forward(const at::Tensor& hidden, const at::Tensor& local_ids, const at::Tensor& weights,
                 const at::Tensor& valid_count, const at::Tensor& w13, const at::Tensor& w2, at::Tensor& partial,
                 at::Tensor& sorted_row, at::Tensor& sorted_scale, at::Tensor& entry_pos, at::Tensor& tile_expert,
                 at::Tensor& counters, at::Tensor& error_flag, const std::optional<at::Tensor>& sorted_x_opt,
                 at::Tensor& act, at::Tensor& y, int64_t stream_handle, bool pair) {
  // Without a `sorted_x` workspace the first GEMM gathers its activation rows itself (TMA gather
  // copies driven by `sorted_row`); with one, a gather kernel permutes them first.
  const bool gathered = !sorted_x_opt.has_value();
  at::Tensor sorted_x = gathered ? hidden : *sorted_x_opt;
  expect(hidden, at::kBFloat16, "hidden");
  expect(local_ids, at::kLong, "local_ids");
  expect(weights, at::kFloat, "weights");
  expect(valid_count, at::kInt, "valid_count");
  expect(w13, at::kBFloat16, "w13");
  expect(w2, at::kBFloat16, "w2");
  expect(partial, at::kBFloat16, "partial");
  expect(sorted_row, at::kInt, "sorted_row");
  expect(sorted_scale, at::kFloat, "sorted_scale");
  expect(entry_pos, at::kInt, "entry_pos");
  expect(tile_expert, at::kInt, "tile_expert");
  expect(counters, at::kInt, "counters");
  expect(error_flag, at::kInt, "error_flag");
  if (sorted_x_opt.has_value()) expect(*sorted_x_opt, at::kBFloat16, "sorted_x");
  expect(act, at::kBFloat16, "act");
  expect(y, at::kBFloat16, "y");
  TORCH_CHECK(hidden.dim() == 2 && local_ids.dim() == 2 && w13.dim() == 3 && w2.dim() == 3, "bad ranks");
  const int64_t rows = hidden.size(0), hidden_size = hidden.size(1), topk = local_ids.size(1);
  const int64_t experts = w13.size(0), inter = w13.size(1) / 2;
  TORCH_CHECK(local_ids.size(0) == rows && weights.size(0) == rows && weights.size(1) == topk, "row mismatch");
  TORCH_CHECK(w13.size(2) == hidden_size && w2.size(0) == experts && w2.size(1) == hidden_size && w2.size(2) == inter,
              "w13 must be [experts, 2 * inter, hidden] and w2 [experts, hidden, inter]");
  TORCH_CHECK(hidden_size % 256 == 0 && inter % 128 == 0, "hidden must be a multiple of 256 and inter of 128");
  TORCH_CHECK(partial.size(0) >= rows && partial.size(1) == hidden_size, "partial must be [>= rows, hidden]");
  const int64_t sorted_rows = sorted_row.numel();
  const int tile = pair ? 2 * kMoeTileRows : kMoeTileRows;
  TORCH_CHECK(sorted_rows % tile == 0 && sorted_scale.numel() == sorted_rows, "sorted buffers mismatch");
  TORCH_CHECK(entry_pos.numel() >= rows * topk && counters.numel() >= 2 && error_flag.numel() >= 1, "small buffers");
  TORCH_CHECK(tile_expert.numel() >= sorted_rows / tile, "tile_expert is too small");
  TORCH_CHECK((gathered || sorted_x.numel() >= sorted_rows * hidden_size) && y.numel() >= sorted_rows * hidden_size &&
              act.numel() >= sorted_rows * inter, "workspace tensors are too small");
  TORCH_CHECK(!gathered || (reinterpret_cast<uintptr_t>(hidden.data_ptr()) % 16 == 0 && rows > 0),
              "gathered loads need a 16-byte aligned, non-empty activation matrix");
  c10::cuda::CUDAGuard guard(hidden.device());
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_handle);
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int max_tiles = static_cast<int>(sorted_rows / tile);
  check(launch_moe_align(reinterpret_cast<const long long*>(local_ids.data_ptr<int64_t>()), weights.data_ptr<float>(),
                         valid_count.data_ptr<int>(), static_cast<int>(rows), static_cast<int>(topk),
                         static_cast<int>(experts), sorted_rows, max_tiles, sorted_row.data_ptr<int>(),
                         sorted_scale.data_ptr<float>(), entry_pos.data_ptr<int>(), tile_expert.data_ptr<int>(),
                         counters.data_ptr<int>(), error_flag.data_ptr<int>(), tile, stream), "align");
  if (!gathered)
    check(launch_moe_gather(hidden.data_ptr(), sorted_row.data_ptr<int>(), counters.data_ptr<int>(), sorted_x.data_ptr(),
                            sorted_rows, static_cast<int>(hidden_size), stream), "gather");
  check(launch_moe_gemm_gate_up(sorted_x.data_ptr(), w13.data_ptr(), act.data_ptr(), counters.data_ptr<int>(),
                                tile_expert.data_ptr<int>(), error_flag.data_ptr<int>(), sorted_rows,
                                static_cast<int>(experts), static_cast<int>(hidden_size), static_cast<int>(inter), sms,
                                pair, stream, gathered ? sorted_row.data_ptr<int>() : nullptr, gathered ? rows : 0),
        "gate/up GEMM");
  check(launch_moe_gemm_down(act.data_ptr(), w2.data_ptr(), y.data_ptr(), sorted_scale.data_ptr<float>(),
                             counters.data_ptr<int>(), tile_expert.data_ptr<int>(), error_flag.data_ptr<int>(),
                             sorted_rows, static_cast<int>(experts), static_cast<int>(hidden_size),
                             static_cast<int>(inter), sms, pair, stream), "down GEMM");
  check(launch_moe_slot_sum(y.data_ptr(), entry_pos.data_ptr<int>(), valid_count.data_ptr<int>(), partial.data_ptr(),
                            static_cast<int>(rows), static_cast<int>(topk), static_cast<int>(hidden_size), stream),
        "slot sum");
}

}  // namespace

void bind_moe(py::module_& m) {
  m.def("moe_sizes", [](int64_t rows, int topk, int experts, int tile_rows) {
    const MoeSizes s = moe_sizes(rows, topk, experts, tile_rows);
    return py::make_tuple(s.max_sorted_rows, s.max_tiles);
  }, py::arg("rows"), py::arg("topk"), py::arg("experts"), py::arg("tile_rows") = kMoeTileRows);
  m.def("moe_forward", &moe_forward);
  m.attr("MOE_TILE_ROWS") = kMoeTileRows;
}

}  // namespace epx
