// GPU helpers of the host-staged transport: a registry of page-locked host ranges, a
// bounds-checked device-to-host copy into such a range, and the two kernels of its combine.
//
// Counterparts of the reference's registration registry and host-CE helper kernels
// (ep_xpress/csrc/bindings.cpp:39-123, ep_xpress/csrc/kernels.cu:13-36): `add_partial`
// accumulates BF16 partial rows into an FP32 plane at given token indices (unique indices,
// no atomics), `finish_combine` rounds the remote sum to BF16, adds the local row and rounds
// again. Differences: an index outside the plane sets a status word and skips the row instead
// of raising a device assert (nothing here may trap a shared GPU), and `finish_combine` also
// knows the single-rounding formula of the multi-node transport.
#include "host_helpers.h"

#include <cuda_bf16.h>

#include <map>
#include <mutex>
#include <stdexcept>
#include <string>

#include "epx_device.cuh"

namespace epx {
namespace {

struct HostRange {
  size_t bytes;
};
std::mutex g_mutex;
std::map<uintptr_t, HostRange> g_ranges;

void check(cudaError_t err, const char* what) {
  if (err != cudaSuccess)
    throw std::runtime_error(std::string("ep_xpress_b200 host helpers: ") + what + ": " + cudaGetErrorString(err));
}

__global__ void __launch_bounds__(256) add_partial_kernel(float* __restrict__ accum, const unsigned short* __restrict__ partial,
                                                          const long long* __restrict__ index, long long rows,
                                                          long long tokens, int hidden, int* status) {
  const long long total = rows * hidden;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long row = i / hidden, column = i - row * hidden;
    const long long token = index[row];
    if (token < 0 || token >= tokens) {
      if (column == 0) atomicExch(status, kInvalidRoute);
      continue;
    }
    float* cell = accum + token * hidden + column;
    *cell = __fadd_rn(*cell, bf16_bits_to_float(partial[i]));
  }
}

__global__ void __launch_bounds__(256) finish_combine_kernel(const float* __restrict__ remote, const float* __restrict__ local,
                                                             unsigned short* __restrict__ out, long long elements,
                                                             int single_round) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < elements; i += stride) {
    float sum = remote[i];
    if (!single_round) sum = __fadd_rn(bf16_bits_to_float(float_to_bf16_bits(sum)), local[i]);
    out[i] = float_to_bf16_bits(sum);
  }
}

int grid_for(long long elements) {
  const long long ctas = (elements + 255) / 256;
  return static_cast<int>(ctas < 1 ? 1 : (ctas > 4096 ? 4096 : ctas));
}

}  // namespace

void register_host_range(void* address, size_t bytes) {
  if (address == nullptr || bytes == 0) throw std::invalid_argument("a host range needs an address and a size");
  const uintptr_t begin = reinterpret_cast<uintptr_t>(address);
  std::lock_guard<std::mutex> lock(g_mutex);
  auto next = g_ranges.lower_bound(begin);
  if (next != g_ranges.end() && next->first < begin + bytes)
    throw std::invalid_argument("host range overlaps a registered range");
  if (next != g_ranges.begin()) {
    auto prev = std::prev(next);
    if (prev->first + prev->second.bytes > begin) throw std::invalid_argument("host range overlaps a registered range");
  }
  check(cudaHostRegister(address, bytes, cudaHostRegisterPortable), "cudaHostRegister");
  g_ranges[begin] = HostRange{bytes};
}

void unregister_host_range(void* address) {
  std::lock_guard<std::mutex> lock(g_mutex);
  auto it = g_ranges.find(reinterpret_cast<uintptr_t>(address));
  if (it == g_ranges.end()) throw std::invalid_argument("address is not the start of a registered host range");
  g_ranges.erase(it);
  check(cudaHostUnregister(address), "cudaHostUnregister");
}

size_t registered_host_ranges() {
  std::lock_guard<std::mutex> lock(g_mutex);
  return g_ranges.size();
}

void check_host_range(const void* address, size_t bytes) {
  const uintptr_t begin = reinterpret_cast<uintptr_t>(address);
  std::lock_guard<std::mutex> lock(g_mutex);
  auto it = g_ranges.upper_bound(begin);
  if (it != g_ranges.begin()) {
    --it;
    if (begin >= it->first && begin + bytes <= it->first + it->second.bytes) return;
  }
  throw std::out_of_range("destination is not inside a registered host range");
}

cudaError_t copy_device_to_registered_host(const void* device_source, void* host_destination, size_t bytes,
                                           cudaStream_t stream) {
  check_host_range(host_destination, bytes);
  return cudaMemcpyAsync(host_destination, device_source, bytes, cudaMemcpyDeviceToHost, stream);
}

cudaError_t launch_add_partial(float* accum, const void* partial, const long long* index, long long rows,
                               long long tokens, int hidden, int* status, cudaStream_t stream) {
  if (rows <= 0 || hidden <= 0) return cudaSuccess;
  add_partial_kernel<<<grid_for(rows * hidden), 256, 0, stream>>>(accum, static_cast<const unsigned short*>(partial),
                                                                  index, rows, tokens, hidden, status);
  return cudaGetLastError();
}

cudaError_t launch_finish_combine(const float* remote, const float* local, void* out, long long elements,
                                  bool single_round, cudaStream_t stream) {
  if (elements <= 0) return cudaSuccess;
  finish_combine_kernel<<<grid_for(elements), 256, 0, stream>>>(remote, local, static_cast<unsigned short*>(out),
                                                                elements, single_round ? 1 : 0);
  return cudaGetLastError();
}

}  // namespace epx
