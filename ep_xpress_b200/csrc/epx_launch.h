// Host-callable launchers of the transport kernels (plain C++, no torch types).
#pragma once
#include <cuda_runtime.h>
#include "epx_layout.h"

namespace epx {

// Dynamic shared memory of the dispatch kernel for a launch of at most `max_tokens` local
// tokens: the per-tile prefix table, then (16-byte rows only) the movers' stage rings, which
// start at `dispatch_ring_offset`.
size_t dispatch_ring_offset(int max_tokens, int world);
size_t dispatch_dynamic_smem(int max_tokens, int world, bool vec16);

// Largest number of CTAs of each kernel that can be resident at once on the
// current device; a cooperative launch may not exceed it. (The reference
// negotiates the same bound through an occupancy query,
// ep_xpress/csrc/host_sm.cu:2516-2564.)
cudaError_t dispatch_max_ctas(bool ids64, bool vec16, size_t dynamic_smem, int* ctas);
cudaError_t combine_max_ctas(bool vec16, int fanout, int* ctas);

// `cooperative` selects cudaLaunchCooperativeKernel (the driver guarantees that all CTAs are
// resident together) over a plain launch (cheaper to enqueue; co-residency then rests on the
// grid fitting the device, which the caller bounds with the *_max_ctas queries, and on no
// other kernel holding the SMs forever).
cudaError_t launch_dispatch(const DispatchArgs& args, int ranks, int ctas_per_rank, bool ids64, bool vec16,
                            size_t dynamic_smem, bool cooperative, cudaStream_t stream);
// `mailbox`: push and reduce run side by side in every CTA (pusher warps move rows with bulk
// copies and release one arrival word per row; the other warps reduce a token as soon as the
// rows it is owed are in) instead of one after the other. It applies to 16-byte rows, fan-outs
// up to eight, rows of up to 112 KiB and groups of two or more ranks (`combine_can_mailbox`); elsewhere, and when not
// asked for, the sequential protocol runs. All ranks of a group must choose the same protocol.
bool combine_can_mailbox(bool vec16, int fanout, int world, long long row_bytes);
cudaError_t launch_combine(const CombineArgs& args, int ranks, int ctas_per_rank, bool vec16, int fanout, int world,
                           int hidden, bool mailbox, bool cooperative, cudaStream_t stream);

// Synthetic expert used by the validation harness and the communication
// benchmark: partial[row] = bf16(hidden[row] * sum_k weights[row,k] * factor[local_ids[row,k]])
// over slots with local_ids >= 0, for rows below *valid_count.
cudaError_t launch_scale_rows(const void* hidden, const long long* local_ids, const float* weights,
                              const int* valid_count, const float* factors, int num_factors, void* partial,
                              int capacity, int hidden_size, int topk, cudaStream_t stream);

// Resets the rows of a fresh slot to the padding state (ids -1, weights 0,
// inverse -1, zero activations) and clears its bookkeeping words.
cudaError_t launch_slot_reset(char* slot, SlotLayout layout, long long capacity, int hidden, int topk,
                              cudaStream_t stream);

}  // namespace epx
