// GPU-side helpers of the host-staged transport (plain C++, no torch types); see host_helpers.cu.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace epx {

// Page-locks [address, address + bytes) and records it; overlapping ranges are rejected.
void register_host_range(void* address, size_t bytes);
void unregister_host_range(void* address);
size_t registered_host_ranges();
// Throws unless the range lies inside one registered range.
void check_host_range(const void* address, size_t bytes);
// Asynchronous device-to-host copy whose destination must lie inside a registered range.
cudaError_t copy_device_to_registered_host(const void* device_source, void* host_destination, size_t bytes,
                                           cudaStream_t stream);
// accum[index[row], :] += float(partial[row, :]) in FP32 (indices are unique per call; an index
// outside [0, tokens) sets *status to 1 and skips the row).
cudaError_t launch_add_partial(float* accum, const void* partial, const long long* index, long long rows,
                               long long tokens, int hidden, int* status, cudaStream_t stream);
// out = bf16(float(bf16(remote)) + local), or bf16(remote) with `single_round`.
cudaError_t launch_finish_combine(const float* remote, const float* local, void* out, long long elements,
                                  bool single_round, cudaStream_t stream);

}  // namespace epx
