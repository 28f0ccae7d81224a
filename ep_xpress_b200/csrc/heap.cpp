// Registry of this process's peer-mapped heaps: allocation, CUDA IPC export/open, and bounds
// checks of every range a launch is given. Plays the role of the reference's overlap-checked
// registry of cudaHostRegister'ed ranges (ep_xpress/csrc/bindings.cpp:39-99) for device memory.
#include "heap.h"

#include <cuda_runtime.h>

#include <cstring>
#include <stdexcept>

namespace epx {
namespace {

void check(cudaError_t err, const char* what) {
  if (err != cudaSuccess)
    throw std::runtime_error(std::string("ep_xpress_b200 heap: ") + what + ": " + cudaGetErrorString(err));
}

}  // namespace

HeapRegistry& HeapRegistry::instance() {
  static HeapRegistry registry;
  return registry;
}

void* HeapRegistry::allocate(size_t bytes) {
  if (bytes == 0) throw std::invalid_argument("heap size must be positive");
  int device = -1;
  check(cudaGetDevice(&device), "cudaGetDevice");
  void* base = nullptr;
  check(cudaMalloc(&base, bytes), "cudaMalloc of the peer-mapped heap");
  cudaError_t err = cudaMemset(base, 0, bytes);
  if (err == cudaSuccess) err = cudaDeviceSynchronize();
  if (err != cudaSuccess) {
    cudaFree(base);
    check(err, "zero-filling the heap");
  }
  std::lock_guard<std::mutex> lock(mutex_);
  mappings_[reinterpret_cast<uintptr_t>(base)] = HeapMapping{base, bytes, true, device};
  return base;
}

std::string HeapRegistry::export_handle(void* base) {
  {
    std::lock_guard<std::mutex> lock(mutex_);
    auto it = mappings_.find(reinterpret_cast<uintptr_t>(base));
    if (it == mappings_.end() || !it->second.owned)
      throw std::invalid_argument("only a heap allocated by this process can be exported");
  }
  cudaIpcMemHandle_t handle;
  check(cudaIpcGetMemHandle(&handle, base), "cudaIpcGetMemHandle");
  return std::string(reinterpret_cast<const char*>(&handle), sizeof(handle));
}

void* HeapRegistry::open(const std::string& handle, size_t bytes) {
  if (handle.size() != sizeof(cudaIpcMemHandle_t)) throw std::invalid_argument("malformed IPC handle");
  cudaIpcMemHandle_t raw;
  std::memcpy(&raw, handle.data(), sizeof(raw));
  int device = -1;
  check(cudaGetDevice(&device), "cudaGetDevice");
  void* base = nullptr;
  check(cudaIpcOpenMemHandle(&base, raw, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  std::lock_guard<std::mutex> lock(mutex_);
  const uintptr_t begin = reinterpret_cast<uintptr_t>(base);
  auto next = mappings_.lower_bound(begin);
  const bool overlaps_next = next != mappings_.end() && next->first < begin + bytes;
  bool overlaps_prev = false;
  if (next != mappings_.begin()) {
    auto prev = std::prev(next);
    overlaps_prev = prev->first + prev->second.bytes > begin;
  }
  if (overlaps_next || overlaps_prev) {
    cudaIpcCloseMemHandle(base);
    throw std::runtime_error("peer heap mapping overlaps a live mapping");
  }
  mappings_[begin] = HeapMapping{base, bytes, false, device};
  return base;
}

void HeapRegistry::release(void* base) {
  HeapMapping mapping;
  {
    std::lock_guard<std::mutex> lock(mutex_);
    auto it = mappings_.find(reinterpret_cast<uintptr_t>(base));
    if (it == mappings_.end()) throw std::invalid_argument("address is not the base of a live heap mapping");
    mapping = it->second;
    mappings_.erase(it);
  }
  if (mapping.owned) check(cudaFree(mapping.base), "cudaFree");
  else check(cudaIpcCloseMemHandle(mapping.base), "cudaIpcCloseMemHandle");
}

void HeapRegistry::check_range(const void* address, size_t bytes) const {
  const uintptr_t begin = reinterpret_cast<uintptr_t>(address);
  std::lock_guard<std::mutex> lock(mutex_);
  auto it = mappings_.upper_bound(begin);
  if (it != mappings_.begin()) {
    --it;
    if (begin >= it->first && begin + bytes <= it->first + it->second.bytes) return;
  }
  throw std::out_of_range("range is not inside a live heap mapping");
}

size_t HeapRegistry::live_mappings() const {
  std::lock_guard<std::mutex> lock(mutex_);
  return mappings_.size();
}

}  // namespace epx
