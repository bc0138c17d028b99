// dl_paged_attention_decode_noalloc: split-KV decode attention for callers that cannot allocate.
//
// This entry point has no counterpart in dynalm-project/dynalm; it exists for users of this library.
//
// Who cannot allocate: code that calls these kernels through the C symbols without a tensor library
// behind it (a C, C++, Go or Rust host, a plugin inside somebody else's server) and that either runs
// where cudaMalloc is forbidden or far too slow (cudaMalloc synchronises the whole device, so it has no
// place on a per-token latency path), or whose device memory was handed out to the last byte by the
// host application at start-up, so that no allocator is left to ask. Such a caller can pass its inputs and
// its output, but has nowhere to get the scratch that the split-KV kernel needs for its partial results.
//
// What it does instead: the scratch lives in a file-scope `static __device__` array inside the library,
// DL_NOALLOC_SCRATCH_FLOATS floats (4 MiB) on every GPU that loads the library, held until the process
// exits. The entry point is otherwise the tensor-core split-KV kernel of attention_decode.cu with the same
// arguments as dl_paged_attention_decode_tc, minus `part`.
//
// Rules:
//  * A call with n_split > 1 is counted as rows * n_heads * n_split * (head_dim + 2) floats of scratch. More
//    than DL_NOALLOC_SCRATCH_FLOATS is refused with DL_ERR_NOALLOC_TOO_LARGE before anything is launched;
//    lower n_split (1 needs no scratch at all) or call per group of rows. The count is made for every call,
//    also for those (2, 4 or 8 splits) whose splits the kernel merges inside a thread-block cluster and which in
//    the end do not touch the array.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
//    device current) and keeps it. That first call should come before any stream capture begins.
//  * All calls on a device share the one array and it keeps what the last call left. Nothing in it has to
//    start at zero: every (row, head, split) record is written by the call before the call reads it.
//    Two calls that overlap on the GPU (different streams, no dependency between them) race on it; run
//    them on one stream or order them with events.
//  * It calls no cudaMalloc, no cudaFree and no library routine that allocates.
#pragma once

#include <cuda_runtime.h>

#define DL_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define DL_ERR_NOALLOC_TOO_LARGE 10002

#ifdef __cplusplus
extern "C" {
#endif

// bfloat16 q / out / cache; see dl_paged_attention_decode_tc for every argument. Returns 0, a cudaError_t,
// DL_ERR_UNSUPPORTED (10001) for sizes the kernel does not take, or DL_ERR_NOALLOC_TOO_LARGE.
int dl_paged_attention_decode_noalloc(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                      const int* block_table, int max_blocks, const int* positions,
                                      const int* row_request, void* out, int out_stride, int rows, int n_heads,
                                      int n_kv_heads, int head_dim, int page_size, float scale, int window,
                                      int n_split, cudaStream_t stream);

// A sentence for a return code of the call above.
const char* dl_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
