// Host-callable launchers of the transport kernels (plain C++, no torch types).
#pragma once
#include <cuda_runtime.h>
#include "epx_layout.h"

namespace epx {

// Dynamic shared memory of the dispatch kernel for a slot laid out for
// `max_tokens` local tokens.
size_t dispatch_dynamic_smem(int max_tokens, int world);

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
// `streamed`: push and reduce run side by side in every CTA (a few warps push while the others
// already reduce the tokens whose rows have arrived) instead of one after the other. Opt-in:
// on B200 the sequential order measured faster (2 GPUs, 4096 tokens: 154 us against 161 us),
// because progress can only be published behind a system-scope fence and that fence does not
// complete while the same SM keeps storing to a peer. It is ignored where the bulk-copy reduce
// does not apply (`combine_can_stream`). Every rank may choose on its own: the progress words
// that peers exchange are the same in both modes.
bool combine_can_stream(bool vec16, int fanout);
cudaError_t launch_combine(const CombineArgs& args, int ranks, int ctas_per_rank, bool vec16, int fanout,
                           bool streamed, bool cooperative, cudaStream_t stream);

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
