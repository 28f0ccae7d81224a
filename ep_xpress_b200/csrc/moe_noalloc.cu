// Allocation-free variant of the grouped SwiGLU expert runner; see moe_noalloc.h for the
// contract. The workspace that `moe_forward` receives as tensors lives here in one
// file-scope device array. Host code may not pass the array's NAME to a kernel (on the
// host it is only a stand-in symbol, not a device address): its device address is
// resolved once per device with cudaGetSymbolAddress and carved up below.
#include "moe_noalloc.h"

#include <cstdint>
#include <mutex>

#include "moe_gemm.h"

namespace {

constexpr long long kSortedRows = 1024;
constexpr long long kMaxPairs = 8192;
constexpr int kMaxHidden = 1024;
constexpr int kMaxInter = 512;
constexpr int kMaxDevices = 64;

constexpr size_t align256(size_t v) { return (v + 255) / 256 * 256; }

// Offsets of the sub-buffers inside the array (all 256-byte aligned).
constexpr size_t kOffSortedRow = 0;                                                    // int32 [kSortedRows]
constexpr size_t kOffSortedScale = kOffSortedRow + align256(kSortedRows * 4);          // f32   [kSortedRows]
constexpr size_t kOffEntryPos = kOffSortedScale + align256(kSortedRows * 4);           // int32 [kMaxPairs]
constexpr size_t kOffTileExpert = kOffEntryPos + align256(kMaxPairs * 4);              // int32 [kSortedRows / 128]
constexpr size_t kOffCounters = kOffTileExpert + align256(kSortedRows / 128 * 4);      // int32 [2] + error flag
constexpr size_t kOffSortedX = kOffCounters + 256;                                     // bf16 [kSortedRows, kMaxHidden]
constexpr size_t kOffAct = kOffSortedX + align256(kSortedRows * kMaxHidden * 2);       // bf16 [kSortedRows, kMaxInter]
constexpr size_t kOffY = kOffAct + align256(kSortedRows * kMaxInter * 2);              // bf16 [kSortedRows, kMaxHidden]
constexpr size_t kScratchBytes = kOffY + align256(kSortedRows * kMaxHidden * 2);

static __device__ __align__(256) unsigned char g_moe_scratch[kScratchBytes];

struct DeviceState {
  unsigned char* scratch = nullptr;
  int sms = 0;
};

std::mutex g_mutex;
DeviceState g_devices[kMaxDevices];

// Set-up of the CURRENT device, once: resolves the device address of the array.
cudaError_t device_state(DeviceState** out) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState& state = g_devices[device];
  if (state.scratch == nullptr) {
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, g_moe_scratch);
    if (err != cudaSuccess) return err;
    int sms = 0;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (err != cudaSuccess) return err;
    state.sms = sms;
    state.scratch = static_cast<unsigned char*>(address);
  }
  *out = &state;
  return cudaSuccess;
}

}  // namespace

extern "C" unsigned long long epx_moe_noalloc_scratch_bytes(void) { return kScratchBytes; }

extern "C" int epx_moe_noalloc_last_status(cudaStream_t stream, int* status, int* cuda_error) {
  if (cuda_error != nullptr) *cuda_error = 0;
  if (status == nullptr) return EPX_NOALLOC_BAD_ARGUMENT;
  auto fail = [&](cudaError_t err) {
    if (cuda_error != nullptr) *cuda_error = static_cast<int>(err);
    return EPX_NOALLOC_CUDA_ERROR;
  };
  DeviceState* state = nullptr;
  cudaError_t err = device_state(&state);
  if (err != cudaSuccess) return fail(err);
  const int* error_flag = reinterpret_cast<const int*>(state->scratch + kOffCounters) + 2;
  err = cudaMemcpyAsync(status, error_flag, sizeof(int), cudaMemcpyDeviceToHost, stream);
  if (err != cudaSuccess) return fail(err);
  err = cudaStreamSynchronize(stream);
  if (err != cudaSuccess) return fail(err);
  return EPX_NOALLOC_OK;
}

extern "C" int epx_moe_forward_noalloc(const void* hidden, const long long* local_ids, const float* weights,
                                       const int* valid_count, const void* w13, const void* w2, void* partial,
                                       int rows, int topk, int experts, int hidden_size, int inter_size,
                                       cudaStream_t stream, int* cuda_error) {
  if (cuda_error != nullptr) *cuda_error = 0;
  if (hidden == nullptr || local_ids == nullptr || weights == nullptr || valid_count == nullptr || w13 == nullptr ||
      w2 == nullptr || partial == nullptr || rows < 0 || topk <= 0 || experts <= 0 || hidden_size <= 0 ||
      inter_size <= 0 || hidden_size % 256 != 0 || inter_size % 128 != 0)
    return EPX_NOALLOC_BAD_ARGUMENT;
  // A misaligned pointer would fault inside a kernel (16-byte vector accesses, TMA): reject it here.
  auto aligned = [](const void* p, uintptr_t to) { return reinterpret_cast<uintptr_t>(p) % to == 0; };
  if (!aligned(hidden, 16) || !aligned(partial, 16) || !aligned(w13, 16) || !aligned(w2, 16) ||
      !aligned(local_ids, 8) || !aligned(weights, 4) || !aligned(valid_count, 4))
    return EPX_NOALLOC_BAD_ARGUMENT;
  const epx::MoeSizes sizes = epx::moe_sizes(rows, topk, experts);
  if (sizes.max_sorted_rows > kSortedRows || static_cast<long long>(rows) * topk > kMaxPairs ||
      hidden_size > kMaxHidden || inter_size > kMaxInter)
    return EPX_NOALLOC_TOO_LARGE;

  auto fail = [&](cudaError_t err) {
    if (cuda_error != nullptr) *cuda_error = static_cast<int>(err);
    return EPX_NOALLOC_CUDA_ERROR;
  };
  DeviceState* state = nullptr;
  cudaError_t err = device_state(&state);
  if (err != cudaSuccess) return fail(err);
  unsigned char* base = state->scratch;
  int* sorted_row = reinterpret_cast<int*>(base + kOffSortedRow);
  float* sorted_scale = reinterpret_cast<float*>(base + kOffSortedScale);
  int* entry_pos = reinterpret_cast<int*>(base + kOffEntryPos);
  int* tile_expert = reinterpret_cast<int*>(base + kOffTileExpert);
  int* counters = reinterpret_cast<int*>(base + kOffCounters);
  int* error_flag = counters + 2;
  void* sorted_x = base + kOffSortedX;
  void* act = base + kOffAct;
  void* y = base + kOffY;

  // The array keeps the previous call's contents: counters and the error flag start at zero.
  // (sorted_row, sorted_scale and entry_pos are rewritten in full by the align step.)
  err = cudaMemsetAsync(counters, 0, 256, stream);
  if (err != cudaSuccess) return fail(err);
  if (rows == 0) return EPX_NOALLOC_OK;
  const long long sorted_rows = sizes.max_sorted_rows;   // <= kSortedRows, a multiple of 128
  err = epx::launch_moe_align(local_ids, weights, valid_count, rows, topk, experts, sorted_rows, sizes.max_tiles,
                              sorted_row, sorted_scale, entry_pos, tile_expert, counters, error_flag,
                              epx::kMoeTileRows, stream);
  if (err != cudaSuccess) return fail(err);
  err = epx::launch_moe_gather(hidden, sorted_row, counters, sorted_x, sorted_rows, hidden_size, stream);
  if (err != cudaSuccess) return fail(err);
  err = epx::launch_moe_gemm_gate_up(sorted_x, w13, act, counters, tile_expert, error_flag, sorted_rows, experts,
                                     hidden_size, inter_size, state->sms, false, stream);
  if (err != cudaSuccess) return fail(err);
  err = epx::launch_moe_gemm_down(act, w2, y, sorted_scale, counters, tile_expert, error_flag, sorted_rows, experts,
                                  hidden_size, inter_size, state->sms, false, stream);
  if (err != cudaSuccess) return fail(err);
  err = epx::launch_moe_slot_sum(y, entry_pos, valid_count, partial, rows, topk, hidden_size, stream);
  if (err != cudaSuccess) return fail(err);
  return EPX_NOALLOC_OK;
}
