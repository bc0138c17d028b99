// y = x W^T on the 5th-generation tensor cores: tcgen05.mma with the accumulator in tensor memory,
// operands brought to shared memory by TMA. bf16 operands, fp32 accumulation.
//
// The kernel and its launcher are in gemm_tcgen05_impl.cuh; this file instantiates them with every block loading
// its own operands (gemm_tcgen05_cluster.cu: with pairs of blocks sharing W tiles).
//
// A thread block computes 128 x BN tiles of y (BN = 256, 192 or 128; for SwiGLU two halves of gate and up
// columns), one after another. Roles (warps 0 and 1 run their loops as whole warps; one elected lane issues):
//   warp 0             TMA producer: for each 64-wide slice of K, waits for a free stage, arms the stage's
//                      mbarrier with the byte count and issues the tile loads (x: 128 rows, W: BN rows), both
//                      K-major with the 128-byte swizzle that the tensor core reads directly
//   warp 1             issues four tcgen05.mma (M 128, N BN, K 16) per stage into the TMEM accumulator and
//                      commits them to the stage's "empty" barrier; after a tile's last slice commits to that
//                      accumulator's "full" barrier. Warp 1 also allocates and frees the TMEM columns.
//   warps 2..5         epilogue: each warp reads its quarter of the 128 TMEM lanes (one output row per thread),
//                      converts and stores: bf16, fp32 (optionally scaled), SwiGLU, where the tile's first
//                      half are gate features and the second the matching up features of W = [Wg; Wu], or the
//                      q | k | v projection's rotary encoding and cache write (qkv_rope.cuh).
// Rows, columns and K past the ends are zero-filled by TMA on the way in and masked on the way out.
//
// Every wait on an mbarrier is bounded: after about a second without progress the waiting role records a code
// in *status, and all roles fall through to the common exit, where the TMEM columns are freed. A block never
// spins forever and never leaves tensor memory allocated.
//
// The reference reaches its GPU matrix products through a library (ggml_mul_mat,
// dynacore/src/gpu/ggml_graph.cpp:278-292) and fuses the gated activation only on its CPU path
// (matmul_gated, dynacore/include/dynacore/device/device.h:188-199).
#include "gemm_tcgen05_impl.cuh"

namespace dl {

// Every block loads its own operands; a stage is free when this block's MMAs have read it.
struct T5Alone {
  static constexpr int CLUSTER = 1;
  static __device__ __forceinline__ void load_shared_half(void*, const CUtensorMap*, int, int, uint64_t*) {}
  static __device__ __forceinline__ void commit_stage_free(uint64_t* bar) { umma_commit(bar); }
};

}  // namespace dl

// The output tile (row block, column block) that tile number `tile` stands for when num_tiles tiles in tiles_n
// columns are numbered in groups of group_m row blocks: the kernel's own numbering, for tests on the host.
DL_EXPORT int dl_gemm_tcgen05_tile_coords(int tile, int tiles_n, int num_tiles, int group_m, int* m_tile, int* n_tile) {
  if (tiles_n <= 0 || num_tiles <= 0 || num_tiles % tiles_n || group_m <= 0 || tile < 0 || tile >= num_tiles) return DL_ERR_UNSUPPORTED;
  dl::t5_tile_coords(tile, tiles_n, num_tiles, group_m, m_tile, n_tile);
  return 0;
}

DL_EXPORT int dl_gemm_tcgen05(const void* x, int ldx, const void* w, void* y, int ldy, int M, int N, int K, int mode,
                              float out_scale, int* status, cudaStream_t stream) {
  if (mode < 0 || mode > 2) return DL_ERR_UNSUPPORTED;
  const dl::QkvRope none = {};
  return t5_launch<dl::T5Alone>(x, ldx, w, y, ldy, M, N, K, mode, out_scale, status, none, stream);
}

// The q | k | v projection with the rotary encoding and the cache write in the epilogue: w bf16 [(n_heads + 2
// n_kv_heads) * head_dim, K], head_dim 64 or 128 with the whole head rotated; rotated q goes to q_out [M, ldq]
// (16-byte aligned rows), rotated k and plain v to the caches [pages, page_size, n_kv_heads, head_dim]. angles:
// [M, head_dim / 2] (cos, sin) pairs from dl_rope_angles, or null (the epilogue then computes them, head by head).
DL_EXPORT int dl_gemm_tcgen05_qkv_rope(const void* x, int ldx, const void* w, void* q_out, int ldq, int M, int K,
                                       const int* positions, const int* row_request, const int* block_table, int max_blocks,
                                       void* k_cache, void* v_cache, const float* inv_freq, const void* angles,
                                       float pos_scale, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                       int* status, cudaStream_t stream) {
  return t5_launch_qkv_rope<dl::T5Alone>(x, ldx, w, q_out, ldq, M, K, positions, row_request, block_table, max_blocks, k_cache,
                                         v_cache, inv_freq, angles, pos_scale, n_heads, n_kv_heads, head_dim, page_size, status,
                                         stream);
}
