// Peer-mapped device heap: one cudaMalloc'd region per rank whose IPC handle is
// exchanged at bootstrap so that every rank of the node can store into and load
// from it over NVLink.
//
// Counterpart of the reference's registration registry for mapped host arenas
// (ep_xpress/csrc/bindings.cpp:39-99): an overlap-checked table of live
// mappings with bounds-checked lookups, except that the mappings are peer HBM,
// not pinned /dev/shm pages.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <mutex>
#include <string>

namespace epx {

struct HeapMapping {
  void* base = nullptr;
  size_t bytes = 0;
  bool owned = false;   // allocated here (cudaFree) vs opened from a peer (cudaIpcCloseMemHandle)
  int device = -1;
};

class HeapRegistry {
 public:
  static HeapRegistry& instance();

  // Allocates `bytes` on the current device and returns the base address. The
  // memory is zero-filled before the call returns.
  void* allocate(size_t bytes);
  // 64-byte CUDA IPC handle of an owned mapping.
  std::string export_handle(void* base);
  // Maps a peer's heap into this process (peer access is enabled lazily).
  void* open(const std::string& handle, size_t bytes);
  // Unmaps / frees one mapping; unknown addresses are rejected.
  void release(void* base);
  // Throws unless [address, address + bytes) lies inside one live mapping.
  void check_range(const void* address, size_t bytes) const;
  size_t live_mappings() const;

 private:
  mutable std::mutex mutex_;
  std::map<uintptr_t, HeapMapping> mappings_;
};

}  // namespace epx
