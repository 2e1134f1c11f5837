// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in willzeng274/kernel-rush-kawk. It exists for
// code that embeds these kernels somewhere cudaMalloc (or any allocating library
// call, torch's caching allocator included) is off limits: inside a region whose
// memory footprint was fixed beforehand, under an allocator that must not be
// re-entered, or in a plug-in that is handed its input and output buffers and
// nothing else. The regular krk_attention_decode needs a float32 scratch buffer from
// its caller for the per-split partial results; this variant keeps that scratch in
// a fixed array inside the library instead, so the caller passes inputs and the
// output only.
//
// Cost and limits
//  * The array is KRK_NOALLOC_SCRATCH_BYTES (4 MiB) of device memory per loaded
//    attention library, held by every GPU that loads the library until the process
//    exits, used or not.
//  * n_seqs * HQ * splits * (head_dim + 2) * 4 bytes must fit in it; a larger
//    request is refused with KRK_NOALLOC_TOO_LARGE and nothing is launched.
//  * The first call on a device looks up the array's device address
//    (cudaGetSymbolAddress) and sets the kernel's shared-memory attribute. Make that
//    first call outside any stream capture.
//  * Head counts and strides are checked before anything else (KRK_NOALLOC_BAD_SHAPE);
//    host threads may call concurrently (the per-device set-up is serialised), but
//    see the next point for what their kernels may not do.
//  * All calls share the one array and it keeps the last call's contents. Nothing
//    in it has to start at zero: every (sequence, head, split) partial is written
//    before the merge reads it. Two calls that overlap on the GPU (different
//    streams without ordering between them) race on the array; order them.
//
// Arguments are those of krk_attention_decode without the scratch pointer:
// out [n_seqs, HQ*D] bfloat16; qkv: row s is sequence s's single new token, its q
// heads first (row stride q_stride elements); seq_slot, seq_start int32 [n_seqs];
// table int32 [slots, width]; k_cache, v_cache [pages, HKV, 64, D] bfloat16.
#pragma once

#include <cuda_runtime.h>

#define KRK_NOALLOC_SCRATCH_BYTES (4u << 20)
#define KRK_NOALLOC_TOO_LARGE (-5)
#define KRK_NOALLOC_SETUP_FAILED (-6)
#define KRK_NOALLOC_BAD_SHAPE (-7)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, a negative KRK_NOALLOC_* / size code, or a positive cudaError_t.
int krk_attention_decode_noalloc(void* out, const void* qkv, int q_stride, int HQ, int HKV, const int* seq_slot,
                                 const int* seq_start, const int* table, int width, const void* k_cache,
                                 const void* v_cache, int n_seqs, float scale, int window, int splits,
                                 cudaStream_t stream);

// A sentence for a return code of the function above.
const char* krk_attention_decode_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
