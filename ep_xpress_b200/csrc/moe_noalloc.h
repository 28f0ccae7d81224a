// Allocation-free entry point of the grouped SwiGLU expert runner.
//
// This entry point has no counterpart in the reference library. It exists for
// callers that cannot allocate device memory at the point where they need the
// experts to run: a latency-critical serving loop in which cudaMalloc (a call
// that synchronises the whole device) is not acceptable, plugins that are handed
// raw device pointers by a host framework and own no allocator, and C callers
// that do not link a tensor library at all. The regular Python
// entry point (`moe_forward`) takes nine caller-provided workspace tensors; this
// one takes only the inputs and the output and keeps its workspace in a
// fixed-size `static __device__` array inside the library.
//
// Limits (checked; a larger problem is rejected with EPX_NOALLOC_TOO_LARGE):
//   (ceil(rows * min(topk, experts) / 128) + experts) * 128 <= 1024 expert-sorted rows
//   (e.g. 640 local (row, slot) pairs over 3 experts), rows * topk <= 8192,
//   hidden_size <= 1024, inter_size <= 512.
// The array is about 5.3 MB per GPU that loads the library, held until the process exits.
//
// The first call on a device resolves the array's device address
// (cudaGetSymbolAddress) and raises the kernels' shared-memory limit; make that first
// call outside any stream capture. Every call reuses the same array: it keeps the
// previous call's contents, the words that must start at zero are cleared on the
// stream at the start of each call, and two calls whose kernels overlap on the GPU
// (different streams without an ordering between them) race on it.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  EPX_NOALLOC_OK = 0,
  EPX_NOALLOC_BAD_ARGUMENT = 1,
  EPX_NOALLOC_TOO_LARGE = 2,
  EPX_NOALLOC_CUDA_ERROR = 3,
};

// partial[row, :] = bf16( sum over the row's local slots, in slot order, of
//                         bf16( (silu(x W1_e) * (x W3_e)) W2_e * weight ) ) for rows < *valid_count.
//   hidden      bf16  [rows, hidden_size]      device
//   local_ids   int64 [rows, topk]             device, -1 = slot not on this rank
//   weights     f32   [rows, topk]             device
//   valid_count int32 [1]                      device
//   w13         bf16  [experts, 2 * inter_size, hidden_size]  device (gate rows, then up rows)
//   w2          bf16  [experts, hidden_size, inter_size]      device
//   partial     bf16  [rows, hidden_size]      device, output
// hidden_size must be a multiple of 256 and inter_size of 128. Alignment (checked on the host,
// nothing is launched when it fails, EPX_NOALLOC_BAD_ARGUMENT): hidden, partial, w13 and w2 on
// 16 bytes (rows are moved as 16-byte vectors and fed to TMA), local_ids on 8, weights and
// valid_count on 4. Returns an EPX_NOALLOC_* code; `cuda_error`, when not null, receives the
// cudaError_t behind EPX_NOALLOC_CUDA_ERROR. EPX_NOALLOC_OK means "enqueued": what the kernels
// found while running is read with epx_moe_noalloc_last_status.
int epx_moe_forward_noalloc(const void* hidden, const long long* local_ids, const float* weights,
                            const int* valid_count, const void* w13, const void* w2, void* partial, int rows,
                            int topk, int experts, int hidden_size, int inter_size, cudaStream_t stream,
                            int* cuda_error);

// Status word that the kernels of the MOST RECENT epx_moe_forward_noalloc call on the current
// device left in the static workspace: 0 = fine, 1 = a bounded wait inside a GEMM gave up (the
// output is incomplete), 2 = more local (row, slot) pairs than the workspace holds (pairs were
// dropped). The word is cleared at the start of every call and shared like the rest of the
// array, so read it before the next call is enqueued. Allocates nothing: the word is copied
// from the array to `*status` on `stream` and the stream is synchronised before returning.
// Returns an EPX_NOALLOC_* code (BAD_ARGUMENT for a null `status`, CUDA_ERROR with the
// cudaError_t in `*cuda_error`); before any forward call on the device the status is 0.
int epx_moe_noalloc_last_status(cudaStream_t stream, int* status, int* cuda_error);

// Size of the library's static workspace in bytes (for documentation and tests).
unsigned long long epx_moe_noalloc_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
