// What the q | k | v projection kernels need to rotate q and k and to write k and v into the paged cache in
// their epilogues (gemm_skinny.cu for few rows, gemm_tcgen05.cu for many). The whole head is rotated (rotary
// width = head_dim); angle, sine and cosine as in rope_cache.cu: theta = float(pos) * pos_scale * inv_freq[i],
// sincosf, fp32. The sums are rounded to bf16 before the rotation, as the unfused path rounds them into its
// q | k | v buffer, so both paths give the same bits.
#pragma once

#include "common.cuh"

namespace dl {

struct QkvRope {
  const int* positions;       // [rows]
  const int* row_request;     // [rows]
  const int* block_table;     // [requests, max_blocks]
  int max_blocks;
  bf16* k_cache;              // [pages, page_size, n_kv_heads, head_dim]
  bf16* v_cache;
  const float* inv_freq;      // [head_dim / 2]
  const float2* angles;       // [rows, head_dim / 2] (cos, sin) from rope_angles_kernel, or null: compute them here
  float pos_scale;
  int n_heads, n_kv_heads, head_dim, page_size;
};

constexpr size_t QKV_NO_SLOT = ~static_cast<size_t>(0);

// The cache slot (page * page_size + offset) of position `pos` of the request in `row`; QKV_NO_SLOT when a
// checked build has refused the request or the page, and the caller then stores neither key nor value.
__device__ __forceinline__ size_t qkv_rope_slot(const QkvRope& p, int row, int pos) {
  const int req = ck_request(p.row_request[row]);
  const int page = ck_page_store(p.block_table + static_cast<size_t>(req) * p.max_blocks, pos / p.page_size, p.max_blocks);
  if (page < 0) return QKV_NO_SLOT;
  return static_cast<size_t>(page) * p.page_size + pos % p.page_size;
}

}  // namespace dl
