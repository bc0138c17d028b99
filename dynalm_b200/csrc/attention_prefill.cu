// Paged flash attention for prompt portions: bf16 tensor cores (mma.sync m16n8k16), fp32 softmax.
//
// One thread block per (query tile, head). A query tile is up to 128 consecutive rows of ONE request
// (the host cuts every request of the step into such tiles; a single decoded token is a tile of one
// row), so portions of several prompts and decode rows share a launch. Keys and values are read in
// place through the request's block table, 64 keys at a time, double-buffered with cp.async; the
// boundaries of those key tiles are multiples of 64 in absolute position, so the arithmetic of a
// row does not depend on where its portion was cut nor on its place inside a query tile.
//
//   S = Q K^T (tensor cores, fp32 accumulators); causal and window mask by position;
//   online softmax in fp32 with base-2 exponentials; O += P V with P rounded to bf16.
//
// Formula and masking as the reference's attention (dynacore/cpu/cpu_device.cpp:1309-1412,
// 1717-1776); the fused softmax.V is where its GPU path calls ggml_flash_attn_ext
// (dynacore/src/gpu/ggml_graph.cpp:465-484), here without a mask tensor.
#include "common.cuh"

namespace dl {

constexpr int PF_TILE = 128;    // rows of a query tile as the host cuts them
constexpr int PF_BN = 64;       // keys per tile
constexpr int PF_THREADS = 128;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the special-function unit: one instruction; 2^-inf = 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

// tiles[i] = (request, first row of the step, rows, first position)
template <int HD>
__global__ void __launch_bounds__(PF_THREADS)
prefill_attention_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ k_cache,
                         const bf16* __restrict__ v_cache, const int* __restrict__ block_table, int max_blocks,
                         const int4* __restrict__ tiles, bf16* __restrict__ out, int out_stride, int n_heads,
                         int n_kv_heads, int page_shift, float scale_log2, int window) {
  // A warp owns PF_MT tiles of 16 query rows and reuses every K and V fragment for all of them. Two tiles per
  // warp were measured slower on B200 at head_dim 64 (235 registers, half as many blocks): one it is.
  constexpr int PF_MT = 1;
  constexpr int PF_BM = 64 * PF_MT;       // query rows per block (4 warps)
  constexpr int SUB = PF_TILE / PF_BM;    // blocks per query tile
  constexpr int LD = HD + 8;              // row stride in elements: 16 bytes of padding keep ldmatrix conflict-free
  constexpr int CH = HD / 8;              // 16-byte chunks per row
  constexpr int KS = HD / 16;             // k-steps of the Q K^T product
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
  bf16* Ks = Qs + PF_BM * LD;             // [2][PF_BN][LD]
  bf16* Vs = Ks + 2 * PF_BN * LD;         // [2][PF_BN][LD]

  const int4 tile = ck_tile(tiles[blockIdx.x / SUB]);
  const int sub = blockIdx.x % SUB;
  const int req = tile.x, row0 = tile.y + sub * PF_BM, nrows = min(PF_BM, tile.z - sub * PF_BM), pos0 = tile.w + sub * PF_BM;
  if (nrows <= 0) return;
  const int head = blockIdx.y;
  const int kvh = head / (n_heads / n_kv_heads);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int page_mask = (1 << page_shift) - 1;
  const int* table = block_table + static_cast<size_t>(req) * max_blocks;
  const size_t kv_row = static_cast<size_t>(n_kv_heads) * HD;

  const int pos_last = pos0 + nrows - 1;
  const int lo_tile = window > 0 ? max(0, pos0 - window + 1) : 0;     // the first key any row of the tile reads
  const int j_begin = lo_tile / PF_BN, j_end = pos_last / PF_BN;

  // Q tile -> shared (rows past the end are zero)
  for (int c = tid; c < PF_BM * CH; c += PF_THREADS) {
    const int r = c / CH, ch = c % CH;
    const bool ok = r < nrows;
    const bf16* src = q + static_cast<size_t>(row0 + (ok ? r : 0)) * q_stride + static_cast<size_t>(head) * HD + ch * 8;
    cp_async16(Qs + r * LD + ch * 8, src, ok);
  }
  // A thread copies the same (row, 16-byte piece) places of every key tile: what does not change from tile to
  // tile is computed once.
  constexpr int KV_ITERS = (PF_BN * CH + PF_THREADS - 1) / PF_THREADS;
  int kv_r[KV_ITERS];                  // key row inside the tile, -1 past the tile
  uint32_t kv_soff[KV_ITERS];          // byte offset inside a stage's K (or V) tile
  size_t kv_goff[KV_ITERS];            // element offset inside a cache row
#pragma unroll
  for (int it = 0; it < KV_ITERS; ++it) {
    const int c = tid + it * PF_THREADS;
    const int r = c / CH, ch = c % CH;
    kv_r[it] = c < PF_BN * CH ? r : -1;
    kv_soff[it] = static_cast<uint32_t>((r * LD + ch * 8) * sizeof(bf16));
    kv_goff[it] = static_cast<size_t>(kvh) * HD + ch * 8;
  }
  const uint32_t ks_base = static_cast<uint32_t>(__cvta_generic_to_shared(Ks));
  const uint32_t vs_base = static_cast<uint32_t>(__cvta_generic_to_shared(Vs));
  auto load_kv = [&](int j, int stage) {
    const uint32_t stage_off = static_cast<uint32_t>(stage * PF_BN * LD * sizeof(bf16));
#pragma unroll
    for (int it = 0; it < KV_ITERS; ++it) {
      if (kv_r[it] < 0) continue;
      const int key = j * PF_BN + kv_r[it];
      const bool ok = key >= lo_tile && key <= pos_last;
      size_t off = 0;
      if (ok) {
        const size_t slot = (static_cast<size_t>(ck_page(table, key >> page_shift, max_blocks)) << page_shift) + (key & page_mask);
        off = slot * kv_row + kv_goff[it];
      }
      const int bytes = ok ? 16 : 0;      // 0 source bytes: the 16 destination bytes are zero-filled
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(ks_base + stage_off + kv_soff[it]), "l"(k_cache + off), "r"(bytes));
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(vs_base + stage_off + kv_soff[it]), "l"(v_cache + off), "r"(bytes));
    }
  };
  load_kv(j_begin, 0);
  cp_async_commit();

  float o[PF_MT][HD / 8][4];
#pragma unroll
  for (int mt = 0; mt < PF_MT; ++mt)
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.0f; }
  float m_run[PF_MT][2], l_run[PF_MT][2];
  int pos_r[PF_MT][2], lo_r[PF_MT][2];            // position and first visible key of the lane's rows
#pragma unroll
  for (int mt = 0; mt < PF_MT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      m_run[mt][h] = -INFINITY;
      l_run[mt][h] = 0.0f;
      pos_r[mt][h] = pos0 + warp * (16 * PF_MT) + mt * 16 + g + h * 8;
      lo_r[mt][h] = window > 0 ? max(0, pos_r[mt][h] - window + 1) : 0;
    }
  uint32_t qf[PF_MT][KS][4];

  for (int j = j_begin; j <= j_end; ++j) {
    const int stage = (j - j_begin) & 1;
    if (j < j_end) load_kv(j + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (j == j_begin) {
      // Q fragments once: the warp's 32 rows, all k-steps
#pragma unroll
      for (int mt = 0; mt < PF_MT; ++mt)
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const int r = warp * (16 * PF_MT) + mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int c = ks * 16 + (lane >> 4) * 8;
          ldmatrix_x4(qf[mt][ks], Qs + r * LD + c);
        }
    }
    const bf16* kt = Ks + stage * PF_BN * LD;
    const bf16* vt = Vs + stage * PF_BN * LD;

    float s[PF_MT][PF_BN / 8][4];
#pragma unroll
    for (int mt = 0; mt < PF_MT; ++mt)
#pragma unroll
      for (int i = 0; i < PF_BN / 8; ++i) { s[mt][i][0] = s[mt][i][1] = s[mt][i][2] = s[mt][i][3] = 0.0f; }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int np = 0; np < PF_BN / 16; ++np) {       // two key tiles of 8 per ldmatrix.x4
        uint32_t kb[4];
        const int key = np * 16 + (lane & 7) + (lane >> 4) * 8;
        const int c = ks * 16 + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(kb, kt + key * LD + c);
#pragma unroll
        for (int mt = 0; mt < PF_MT; ++mt) {
          mma_bf16(s[mt][2 * np], qf[mt][ks], kb[0], kb[1]);
          mma_bf16(s[mt][2 * np + 1], qf[mt][ks], kb[2], kb[3]);
        }
      }
    }
    // scale, mask by position, online softmax; P as bf16 A fragments
    const int key0 = j * PF_BN;
    uint32_t pf[PF_MT][PF_BN / 16][4];
#pragma unroll
    for (int mt = 0; mt < PF_MT; ++mt) {
      const bool edge = key0 + PF_BN - 1 > pos0 + warp * (16 * PF_MT) + mt * 16 ||
                        (window > 0 && key0 < max(lo_r[mt][0], lo_r[mt][1]));
      // Raw scores stay in s; the running maximum is kept in scaled (base-2) units, and the scale is folded
      // into the exponent: p = 2^(s * scale - max).
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < PF_BN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[mt][i][e];
          if (edge) {
            const int key = key0 + i * 8 + 2 * t + (e & 1);
            if (key > pos_r[mt][e >> 1] || key < lo_r[mt][e >> 1]) v = -INFINITY;
            s[mt][i][e] = v;
          }
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
      float corr[2], neg_m[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m_run[mt][h], mx[h] * scale_log2);     // the scale is positive
        // a row with no visible key so far (rows past the end of the tile, or a window that starts
        // later) keeps max = -inf; its probabilities are exact zeros
        corr[h] = m_new == -INFINITY ? 1.0f : fast_exp2(m_run[mt][h] - m_new);
        m_run[mt][h] = m_new;
        neg_m[h] = m_new == -INFINITY ? 0.0f : -m_new;
      }
      float ls[2] = {0.0f, 0.0f};
#pragma unroll
      for (int i = 0; i < PF_BN / 8; ++i) {
        const float p0 = fast_exp2(fmaf(s[mt][i][0], scale_log2, neg_m[0])), p1 = fast_exp2(fmaf(s[mt][i][1], scale_log2, neg_m[0]));
        const float p2 = fast_exp2(fmaf(s[mt][i][2], scale_log2, neg_m[1])), p3 = fast_exp2(fmaf(s[mt][i][3], scale_log2, neg_m[1]));
        ls[0] += p0 + p1;
        ls[1] += p2 + p3;
        pf[mt][i >> 1][(i & 1) * 2] = pack_bf16(p0, p1);
        pf[mt][i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        ls[h] += __shfl_xor_sync(0xffffffffu, ls[h], 1);
        ls[h] += __shfl_xor_sync(0xffffffffu, ls[h], 2);
        l_run[mt][h] = l_run[mt][h] * corr[h] + ls[h];
      }
      // once the maxima have settled the correction is exactly 1 for every row of the warp: skip the rescale
      if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
          o[mt][i][0] *= corr[0]; o[mt][i][1] *= corr[0];
          o[mt][i][2] *= corr[1]; o[mt][i][3] *= corr[1];
        }
      }
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < PF_BN / 16; ++kk) {
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {           // two 8-wide slices of the head dimension per ldmatrix.x4
        uint32_t vb[4];
        const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = dp * 16 + (lane >> 4) * 8;
        ldmatrix_x4_trans(vb, vt + key * LD + c);
#pragma unroll
        for (int mt = 0; mt < PF_MT; ++mt) {
          mma_bf16(o[mt][2 * dp], pf[mt][kk], vb[0], vb[1]);
          mma_bf16(o[mt][2 * dp + 1], pf[mt][kk], vb[2], vb[3]);
        }
      }
    }
    __syncthreads();     // every warp is done with this stage before the next prefetch overwrites it
  }
  cp_async_wait<0>();

#pragma unroll
  for (int mt = 0; mt < PF_MT; ++mt) {
    const int r_a = warp * (16 * PF_MT) + mt * 16 + g, r_b = r_a + 8;
    const float inv_a = l_run[mt][0] > 0.0f ? 1.0f / l_run[mt][0] : 0.0f;
    const float inv_b = l_run[mt][1] > 0.0f ? 1.0f / l_run[mt][1] : 0.0f;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      const int col = head * HD + i * 8 + 2 * t;
      if (r_a < nrows)
        *reinterpret_cast<uint32_t*>(out + static_cast<size_t>(row0 + r_a) * out_stride + col) =
            pack_bf16(o[mt][i][0] * inv_a, o[mt][i][1] * inv_a);
      if (r_b < nrows)
        *reinterpret_cast<uint32_t*>(out + static_cast<size_t>(row0 + r_b) * out_stride + col) =
            pack_bf16(o[mt][i][2] * inv_b, o[mt][i][3] * inv_b);
    }
  }
}

template <int HD>
int launch_prefill(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_blocks,
                   const int* tiles, int n_tiles, void* out, int out_stride, int n_heads, int n_kv_heads, int page_shift,
                   float scale, int window, cudaStream_t stream) {
  constexpr int BM = 64;
  constexpr size_t smem = static_cast<size_t>(BM + 4 * PF_BN) * (HD + 8) * sizeof(bf16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attention_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  dim3 grid(n_tiles * (PF_TILE / BM), n_heads);
  prefill_attention_kernel<HD><<<grid, PF_THREADS, smem, stream>>>(
      static_cast<const bf16*>(q), q_stride, static_cast<const bf16*>(kc), static_cast<const bf16*>(vc), block_table,
      max_blocks, reinterpret_cast<const int4*>(tiles), static_cast<bf16*>(out), out_stride, n_heads, n_kv_heads,
      page_shift, scale * 1.4426950408889634f, window);
  return launch_status();
}

}  // namespace dl

// bfloat16 only. tiles: int32 [n_tiles, 4] = (request, first row, rows <= 128, first position), 16-byte aligned.
// q/out rows have head h at column h * head_dim; both strides and head_dim keep rows 4-byte aligned for the
// packed stores (head_dim is a multiple of 16, at most 128; larger heads take the plain kernel).
DL_EXPORT int dl_paged_attention_prefill(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                         const int* block_table, int max_blocks, const int* tiles, int n_tiles,
                                         void* out, int out_stride, int n_heads, int n_kv_heads, int head_dim,
                                         int page_size, float scale, int window, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  if ((1 << page_shift) != page_size || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_heads > 65535 ||
      (q_stride & 7) || (out_stride & 1) || !(scale > 0.0f))
    return DL_ERR_UNSUPPORTED;
#define DL_CASE(H)                                                                                                  \
  case H:                                                                                                           \
    return dl::launch_prefill<H>(q, q_stride, k_cache, v_cache, block_table, max_blocks, tiles, n_tiles, out,       \
                                 out_stride, n_heads, n_kv_heads, page_shift, scale, window, stream)
  switch (head_dim) {
    DL_CASE(16);
    DL_CASE(32);
    DL_CASE(48);
    DL_CASE(64);
    DL_CASE(80);
    DL_CASE(96);
    DL_CASE(112);
    DL_CASE(128);
    default:
      return DL_ERR_UNSUPPORTED;
  }
#undef DL_CASE
}
