// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for users of this
// library.  Some hosts of a kernel library may not call cudaMalloc at the moment they need a
// kernel: code that runs inside a region where allocation is forbidden or would serialise the
// device (a real-time loop, a callback of another runtime, a process whose memory budget was
// handed out in full at start-up), or code that does not link an allocator at all.  The split
// decode attention needs scratch memory for the partial results of its splits, and the ordinary
// entry point (xrt_attention_decode) expects the caller to bring it.  This one brings its own: a
// fixed array in the library's device image.
//
// What to know before calling it:
//  * The scratch is XRT_DECODE_STATIC_SCRATCH_BYTES (8 MiB) and every GPU that loads the library
//    holds that much until the process exits, used or not.
//  * A call needs n_tokens * n_heads * n_splits * (head_dim + 2) floats of it when n_splits > 1
//    (none when n_splits == 1).  A call that needs more is refused with XRT_ERR_SCRATCH (-3)
//    and a message that names both numbers; nothing is launched.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress) with
//    that device current and keeps it.  Make that first call outside any stream capture.
//  * It allocates nothing and frees nothing: no cudaMalloc, cudaFree or library allocation.
//    Inputs and outputs are the caller's, exactly as for xrt_attention_decode.
//  * All calls share the one array.  It keeps the previous call's contents; nothing in it has to
//    start at zero, because every split that the combine step reads is written first by the same
//    call.  Two calls that overlap on the GPU (different streams, or different threads on the
//    same device) race on it: keep calls on one device in one stream order.
#pragma once

#include <cuda_runtime.h>

#define XRT_DECODE_STATIC_SCRATCH_BYTES (8u << 20)
#define XRT_ERR_SCRATCH -3

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as for xrt_attention_decode without the two scratch pointers: bfloat16 q and out
// [n_tokens, n_heads * head_dim]; bfloat16 pools [blocks, kv heads, 64, head_dim]; int32 tok_slot,
// tok_pos [n_tokens]; int32 block_table [slots, max_blocks]; `chunk` keys a split (a multiple of
// 64), `n_splits` splits.  `message` (may be null) receives a zero-terminated text of at most
// message_len bytes when the call is refused.  Returns 0 when the kernels were launched on
// `stream`, a negative code when the call was refused, a positive cudaError_t otherwise.
__attribute__((visibility("default")))
int xrt_attention_decode_static(void* out, const void* q, const void* k_pool, const void* v_pool,
                                const int* tok_slot, const int* tok_pos, const int* block_table, int max_blocks,
                                int n_tokens, int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                int chunk, int n_splits, cudaStream_t stream, char* message, int message_len);

#ifdef __cplusplus
}
#endif
