// The tcgen05 matrix product with pairs of thread blocks sharing their W tiles (gemm_tcgen05_impl.cuh, P::CLUSTER ==
// 2): a cluster of two blocks computes row blocks 2i and 2i + 1 of one column block; each block loads one half of
// the W tile with a TMA copy that lands in both blocks' shared memory, so every W tile crosses from L2 once per
// pair instead of once per block (a third less operand traffic, which is what bounds the kernel alone).
//
// This file is the only one with a TMA copy that writes into another block's shared memory. It reads this GPU's
// own memory only; the package works without it (kernels/gemm.py then uses gemm_tcgen05.cu).
//
// The reference reaches its GPU matrix products through a library (ggml_mul_mat,
// dynacore/src/gpu/ggml_graph.cpp:278-292).
#include "gemm_tcgen05_impl.cuh"

namespace dl {

struct T5Pair {
  static constexpr int CLUSTER = 2;
  // One half of the pair's W tile into the same place of both blocks' shared memory; the bytes count on the
  // barrier at the same place in each block.
  static __device__ __forceinline__ void load_shared_half(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    const uint16_t both = 0x3;
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.multicast::cluster"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "h"(both) : "memory");
  }
  // The stage is free when both blocks' MMAs have read it: this block's commit arrives on the barrier of both.
  static __device__ __forceinline__ void commit_stage_free(uint64_t* bar) {
    const uint16_t both = 0x3;
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both) : "memory");
  }
};

}  // namespace dl

// As dl_gemm_tcgen05.
DL_EXPORT int dl_gemm_tcgen05_cluster(const void* x, int ldx, const void* w, void* y, int ldy, int M, int N, int K, int mode,
                                      float out_scale, int* status, cudaStream_t stream) {
  if (mode < 0 || mode > 2) return DL_ERR_UNSUPPORTED;
  const dl::QkvRope none = {};
  return t5_launch<dl::T5Pair>(x, ldx, w, y, ldy, M, N, K, mode, out_scale, status, none, stream);
}

// As dl_gemm_tcgen05_qkv_rope.
DL_EXPORT int dl_gemm_tcgen05_cluster_qkv_rope(const void* x, int ldx, const void* w, void* q_out, int ldq, int M, int K,
                                               const int* positions, const int* row_request, const int* block_table,
                                               int max_blocks, void* k_cache, void* v_cache, const float* inv_freq,
                                               const void* angles, float pos_scale, int n_heads, int n_kv_heads, int head_dim,
                                               int page_size, int* status, cudaStream_t stream) {
  return t5_launch_qkv_rope<dl::T5Pair>(x, ldx, w, q_out, ldq, M, K, positions, row_request, block_table, max_blocks, k_cache,
                                        v_cache, inv_freq, angles, pos_scale, n_heads, n_kv_heads, head_dim, page_size, status,
                                        stream);
}
