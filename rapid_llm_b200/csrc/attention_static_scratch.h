// An allocation-free door into the split-key paged attention of attention_mma.cu.
//
// This entry point has no counterpart in harleyszhang/rapid_llm: the reference always lets
// PyTorch's allocator hand its kernels their temporary buffers.
//
// Who needs it.  Some hosts of this library may not create device memory while they run:
// a plug-in inside a process whose memory pool was sized and frozen at start-up, code that
// runs while another component owns the allocator lock, a real-time loop that must not
// risk the implicit device synchronisation of cudaMalloc/cudaFree, or a thin C caller
// that has no allocator of its own at all.  The ordinary entry point, rl_attention_mma,
// asks such a caller for two float32 scratch buffers (the partial outputs and
// log-sum-exps of the key-range splits); this one brings its own.
//
// How.  The scratch is a file-scope `static __device__` array of
// rl_attention_static_scratch_bytes() bytes inside the library image, so every GPU on
// which the library is loaded holds that much memory until the process exits.  The first
// call on a device looks the array's device address up once (cudaGetSymbolAddress, with
// that device current) and remembers it; make that first call outside any stream
// capture.  No call, first or later, uses cudaMalloc, cudaFree or any other allocating
// routine.
//
// Limits and sharing.  The call needs tokens * hq * splits * (head_dim + 1) floats and is
// refused with rl_attention_static_scratch_too_large (see the ..._strerror function) when
// that exceeds the array; nothing is launched then.  All calls on a device use the same
// array and it keeps whatever the previous call left, so the log-sum-exp slots the call
// will read are reset on the stream before the attention kernels run, and the merge skips a
// part whose slot stayed reset (leftovers that are not numbers do no harm either).  Two calls that may
// execute at the same time on one GPU (different streams, no ordering between them) race
// on the array: order them yourself.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Return code, besides cudaError_t values, when the request does not fit the array.
#define RL_ATTENTION_STATIC_SCRATCH_TOO_LARGE (-2)

// Same arguments and result as rl_attention_mma without the two scratch pointers.  With
// splits == 1 no scratch is touched.  Returns 0, a cudaError_t, or
// RL_ATTENTION_STATIC_SCRATCH_TOO_LARGE.
int rl_attention_mma_static_scratch(const void* q, const void* cache, void* out, const int* chunk_items,
                                    int n_chunk_items, const int* decode_items, int n_decode_items,
                                    const int* cu_seqlens, const int* entry_start, const int* entry_slot,
                                    const int* block_table, int tokens, int hq, int hkv, int head_dim,
                                    int page_size, int num_pages, int max_pages, int slots, int window,
                                    int splits, float scale, int* fault, cudaStream_t stream);

// Size of the built-in scratch array in bytes (a compile-time constant of the library).
long long rl_attention_static_scratch_bytes(void);

// A sentence for a code returned by rl_attention_mma_static_scratch.
const char* rl_attention_static_scratch_strerror(int code);

#ifdef __cplusplus
}
#endif
