// y = x W^T for few rows (decode): a weight-streaming matrix product, bf16 operands, fp32 accumulation.
//
// With M <= 64 rows the product is bound by reading W once from HBM, so the kernel is built around
// that stream. It computes y^T = W x^T on the tensor cores (mma.sync m16n8k16): the 16 rows of the
// A operand are 16 output features (rows of W, contiguous in K), the 8 columns of the B operand are 8
// batch rows. A block owns FT = 16 * MT features; its 8 warps split K between them in blocks of 64, each
// lane reading whole 16-byte pieces of a weight row (the k order inside a 32-wide block is permuted
// identically for W and x, which leaves the dot products unchanged), with no shared-memory staging. The
// warps' partial sums are added in shared memory in a fixed order. Small N can also split K over
// gridDim.y blocks, which then write fp32 partial results [split][M][N] that the consumer adds up in a
// fixed order (the residual-add + RMSNorm kernel does), so results never depend on timing.
//
// Epilogues: bf16 or fp32 store, or SwiGLU: W = [Wg; Wu], a block takes 8 gate rows and the 8 matching up
// rows and stores silu(g) * u (the reference's matmul_gated, dynacore/include/dynacore/device/device.h:188-199).
#include "qkv_rope.cuh"

namespace dl {

constexpr int SK_WARPS = 8;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_KB = 64;          // k per block: two 16-byte pieces per lane and row
// Blocks per SM the variants aim for (register caps): four for up to 8 rows; three for 9 to 16 rows, where x
// requested ahead costs 16 registers more (measured, batch 16: 1.17 ms per step against 1.29 ms with two blocks
// and 1.28 ms with four blocks and x not requested ahead).
constexpr int SK_BLOCKS_8 = 4, SK_BLOCKS_16 = 3;

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

enum { SK_OUT_BF16 = 0, SK_OUT_F32 = 1, SK_OUT_SWIGLU = 2, SK_OUT_ARGMAX = 3 };

// The weight stream of one block: y^T tile = W rows (wrow, 16 * MT of them in MMA row order) times x^T, k-blocks
// [blk_begin, blk_end) dealt to the warps round-robin. Leaves every warp's partial tile in `red`
// ([SK_WARPS][MT * 16][NT * 8] floats, shared) and synchronises the block.
template <int MT, int NT>
__device__ __forceinline__ void skinny_accumulate(const bf16* __restrict__ x, int ldx, const bf16* const (&wrow)[MT][2],
                                                  const bool (&wok)[MT][2], int M, int K, int blk_begin, int blk_end,
                                                  float* red, const void* ahead = nullptr, long long ahead_bytes = 0) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const bf16* xrow[NT];
  bool xok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int b = nt * 8 + g;
    xok[nt] = b < M;
    xrow[nt] = x + static_cast<size_t>(xok[nt] ? b : 0) * ldx;
  }
  float acc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.0f; }

  // The weight rows of a k-block: 16-byte pieces at k0 and k0 + 32 of each of the lane's rows.
  const uint4 zero = make_uint4(0, 0, 0, 0);
  auto load_w = [&](int blk, uint4 (&a)[MT][2][2]) {
    const int k0 = blk * SK_KB + 8 * t;
    const bool ok0 = k0 + 8 <= K, ok1 = k0 + 32 + 8 <= K;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        a[mt][h][0] = (wok[mt][h] && ok0) ? ld_stream16(wrow[mt][h] + k0) : zero;
        a[mt][h][1] = (wok[mt][h] && ok1) ? ld_stream16(wrow[mt][h] + k0 + 32) : zero;
      }
  };
  auto load_x = [&](int blk, uint4 (&bq)[NT][2]) {
    const int k0 = blk * SK_KB + 8 * t;
    const bool ok0 = k0 + 8 <= K, ok1 = k0 + 32 + 8 <= K;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      bq[nt][0] = (xok[nt] && ok0) ? *reinterpret_cast<const uint4*>(xrow[nt] + k0) : zero;
      bq[nt][1] = (xok[nt] && ok1) ? *reinterpret_cast<const uint4*>(xrow[nt] + k0 + 32) : zero;
    }
  };
  // The weights do not depend on the kernel before this one: the first pieces are on their way before the wait
  // for it, and each k-block's pieces (weights and x) are requested one block ahead of their use.
  // (x is requested ahead only in the variants for up to 16 rows: more would cost registers.)
  constexpr bool X_AHEAD = NT <= 2;
  uint4 a[MT][2][2], bq[NT][2];
  int blk = blk_begin + warp;
  if (blk < blk_end) load_w(blk, a);
  l2_prefetch_share(ahead, ahead_bytes);     // what the kernel after this one will stream (see common.cuh)
  pdl_wait();
  pdl_trigger();
  if (X_AHEAD && blk < blk_end) load_x(blk, bq);
  for (; blk < blk_end; blk += SK_WARPS) {
    uint4 a_next[MT][2][2], bq_next[X_AHEAD ? NT : 1][2];
    const bool more = blk + SK_WARPS < blk_end;
    if (more) {
      load_w(blk + SK_WARPS, a_next);
      if constexpr (X_AHEAD) load_x(blk + SK_WARPS, bq_next);
    }
    if constexpr (!X_AHEAD) load_x(blk, bq);
#pragma unroll
    for (int c = 0; c < 2; ++c) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          // 16-byte piece = words (x, y, z, w) = k pairs; one mma takes (x, y), the next (z, w)
          mma16816(acc[mt][nt], a[mt][0][c].x, a[mt][1][c].x, a[mt][0][c].y, a[mt][1][c].y, bq[nt][c].x, bq[nt][c].y);
          mma16816(acc[mt][nt], a[mt][0][c].z, a[mt][1][c].z, a[mt][0][c].w, a[mt][1][c].w, bq[nt][c].z, bq[nt][c].w);
        }
      }
    }
    if (more) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) { a[mt][h][0] = a_next[mt][h][0]; a[mt][h][1] = a_next[mt][h][1]; }
      if constexpr (X_AHEAD) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { bq[nt][0] = bq_next[nt][0]; bq[nt][1] = bq_next[nt][1]; }
      }
    }
  }

  // warps -> shared; c0,c1: (feature g, batch 2t, 2t+1); c2,c3: (feature g + 8, same batch)
  constexpr int FT = MT * 16, BT = NT * 8;
  float* mine = red + static_cast<size_t>(warp) * FT * BT;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int b = nt * 8 + 2 * t;
      mine[(mt * 16 + g) * BT + b] = acc[mt][nt][0];
      mine[(mt * 16 + g) * BT + b + 1] = acc[mt][nt][1];
      mine[(mt * 16 + g + 8) * BT + b] = acc[mt][nt][2];
      mine[(mt * 16 + g + 8) * BT + b + 1] = acc[mt][nt][3];
    }
  __syncthreads();
}

// MT: m16 tiles (16 features each) per block; NT: n8 tiles (8 batch rows each).
template <int MT, int NT>
__global__ void __launch_bounds__(SK_THREADS, (MT == 1 && NT <= 2) ? (NT == 1 ? SK_BLOCKS_8 : SK_BLOCKS_16) : 1)
gemm_skinny_kernel(const bf16* __restrict__ x, int ldx, const bf16* __restrict__ w, void* __restrict__ y, int ldy,
                   int M, int N, int K, int mode, float out_scale, long long split_stride,
                   const void* __restrict__ ahead, long long ahead_bytes) {
  extern __shared__ float red[];     // [SK_WARPS][MT * 16][NT * 8]
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int f0 = blockIdx.x * (MT * 16);
  const int n_split = gridDim.y, split = blockIdx.y;
  const int half = N / 2;            // SwiGLU: gate rows [0, half), up rows [half, N)

  // the weight rows of this lane: features f0 + mt*16 + g and + 8
  const bf16* wrow[MT][2];
  bool wok[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int f;
      if (mode == SK_OUT_SWIGLU) {
        const int j = blockIdx.x * (MT * 8) + mt * 8 + g;   // gate row j, up row half + j
        f = h == 0 ? j : half + j;
        wok[mt][h] = j < half;
      } else {
        f = f0 + mt * 16 + g + h * 8;
        wok[mt][h] = f < N;
      }
      wrow[mt][h] = w + static_cast<size_t>(wok[mt][h] ? f : 0) * K;
    }
  }
  // K range of this block, in blocks of 64
  const int nblk = (K + SK_KB - 1) / SK_KB;
  const int per = (nblk + n_split - 1) / n_split;
  const int blk_begin = split * per, blk_end = min(nblk, blk_begin + per);
  skinny_accumulate<MT, NT>(x, ldx, wrow, wok, M, K, blk_begin, blk_end, red, ahead, ahead_bytes);

  constexpr int FT = MT * 16, BT = NT * 8;
  if (mode == SK_OUT_SWIGLU) {
    // tile rows [mt*16 + i] = gate j, [mt*16 + 8 + i] = up j, j = blockIdx.x * MT*8 + mt*8 + i
    for (int idx = threadIdx.x; idx < MT * 8 * BT; idx += SK_THREADS) {
      const int b = idx / (MT * 8), jj = idx % (MT * 8);
      const int mt = jj / 8, i = jj % 8;
      const int j = blockIdx.x * (MT * 8) + jj;
      if (b >= M || j >= half) continue;
      float gate = 0.0f, up = 0.0f;
#pragma unroll
      for (int wv = 0; wv < SK_WARPS; ++wv) {
        gate += red[(static_cast<size_t>(wv) * FT + mt * 16 + i) * BT + b];
        up += red[(static_cast<size_t>(wv) * FT + mt * 16 + 8 + i) * BT + b];
      }
      const float s = gate / (1.0f + expf(-gate));
      static_cast<bf16*>(y)[static_cast<size_t>(b) * ldy + j] = __float2bfloat16_rn(s * up);
    }
    return;
  }
  if (mode == SK_OUT_ARGMAX) {
    // no logits leave the block: per batch row the largest of its FT features and where it is (the lowest feature
    // among equals), into y as float [M][blocks] followed by int [M][blocks]; a small kernel picks among the blocks
    const int blocks = gridDim.x;
    float* pv = static_cast<float*>(y);
    int* pi = reinterpret_cast<int*>(pv + static_cast<size_t>(M) * blocks);
    for (int b = threadIdx.x; b < M; b += SK_THREADS) {
      float best = -INFINITY;
      int where = 0x7fffffff;
      for (int fi = 0; fi < FT; ++fi) {
        if (f0 + fi >= N) break;
        float v = 0.0f;
#pragma unroll
        for (int wv = 0; wv < SK_WARPS; ++wv) v += red[(static_cast<size_t>(wv) * FT + fi) * BT + b];
        v *= out_scale;
        if (v > best) { best = v; where = f0 + fi; }
      }
      pv[static_cast<size_t>(b) * blocks + blockIdx.x] = best;
      pi[static_cast<size_t>(b) * blocks + blockIdx.x] = where;
    }
    return;
  }
  for (int idx = threadIdx.x; idx < FT * BT; idx += SK_THREADS) {
    const int b = idx / FT, fi = idx % FT;      // consecutive threads -> consecutive features of one batch row
    const int f = f0 + fi;
    if (b >= M || f >= N) continue;
    float v = 0.0f;
#pragma unroll
    for (int wv = 0; wv < SK_WARPS; ++wv) v += red[(static_cast<size_t>(wv) * FT + fi) * BT + b];
    v *= out_scale;
    if (mode == SK_OUT_F32)
      static_cast<float*>(y)[static_cast<size_t>(split) * split_stride + static_cast<size_t>(b) * ldy + f] = v;
    else
      static_cast<bf16*>(y)[static_cast<size_t>(b) * ldy + f] = __float2bfloat16_rn(v);
  }
}

// The q | k | v projection of an attention layer with the rotary encoding and the cache write in its epilogue.
// W = [Wq; Wk; Wv]. A block of a q or k head takes 8 rotary pairs: its 16 MMA rows are features p .. p + 7 and
// p + half .. p + half + 7 of the head (half = head_dim / 2: the whole head is rotated), so both members of a
// pair meet in one block. A block of a v head takes 16 consecutive features. The sums are rounded to bf16
// before the rotation, as the unfused path rounds them into its q | k | v buffer; the rotation is the one of
// rope_cache.cu (same angle formula, sincosf, fp32), so both paths give the same bits. Rotated q goes to
// q_out [M, ldq], rotated k and plain v into the request's cache page.
template <int NT>
__global__ void __launch_bounds__(SK_THREADS, NT == 1 ? SK_BLOCKS_8 : SK_BLOCKS_16)
gemm_skinny_qkv_rope_kernel(const bf16* __restrict__ x, int ldx, const bf16* __restrict__ w, bf16* __restrict__ q_out,
                            int ldq, int M, int K, QkvRope p) {
  extern __shared__ float red[];     // [SK_WARPS][16][NT * 8]
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int hd = p.head_dim, half = hd / 2, per_head = hd / 16;
  const int rot_blocks = (p.n_heads + p.n_kv_heads) * per_head;
  const bool rotated = static_cast<int>(blockIdx.x) < rot_blocks;
  int head, f_lo, f_hi;              // head counts q heads, then k heads, then v heads
  if (rotated) {
    head = blockIdx.x / per_head;
    f_lo = head * hd + (blockIdx.x % per_head) * 8;
    f_hi = f_lo + half;
  } else {
    const int vb = blockIdx.x - rot_blocks;
    head = p.n_heads + p.n_kv_heads + vb / per_head;
    f_lo = head * hd + (vb % per_head) * 16;
    f_hi = f_lo + 8;
  }
  const bf16* wrow[1][2] = {{w + static_cast<size_t>(f_lo + g) * K, w + static_cast<size_t>(f_hi + g) * K}};
  const bool wok[1][2] = {{true, true}};
  skinny_accumulate<1, NT>(x, ldx, wrow, wok, M, K, 0, (K + SK_KB - 1) / SK_KB, red);

  constexpr int BT = NT * 8;
  for (int idx = threadIdx.x; idx < 8 * BT; idx += SK_THREADS) {
    const int b = idx / 8, i = idx % 8;
    if (b >= M) continue;
    float lo = 0.0f, hi = 0.0f;
#pragma unroll
    for (int wv = 0; wv < SK_WARPS; ++wv) {
      lo += red[(static_cast<size_t>(wv) * 16 + i) * BT + b];
      hi += red[(static_cast<size_t>(wv) * 16 + 8 + i) * BT + b];
    }
    lo = __bfloat162float(__float2bfloat16_rn(lo));
    hi = __bfloat162float(__float2bfloat16_rn(hi));
    const int pos = p.positions[b];
    bf16* dst;                       // where feature f_lo + i of row b goes; f_hi + i lies (f_hi - f_lo) further
    if (rotated) {
      const float theta = static_cast<float>(pos) * p.pos_scale * p.inv_freq[f_lo - head * hd + i];
      float sn, c;
      sincosf(theta, &sn, &c);
      const float ra = lo * c - hi * sn, rb = lo * sn + hi * c;
      lo = ra;
      hi = rb;
    }
    if (head < p.n_heads) {
      dst = q_out + static_cast<size_t>(b) * ldq + f_lo + i;
    } else {
      const size_t slot = qkv_rope_slot(p, b, pos);
      if (slot == QKV_NO_SLOT) continue;
      const bool is_k = head < p.n_heads + p.n_kv_heads;
      const int kvh = head - p.n_heads - (is_k ? 0 : p.n_kv_heads);
      dst = (is_k ? p.k_cache : p.v_cache) + (slot * p.n_kv_heads + kvh) * hd + (f_lo - head * hd) + i;
    }
    dst[0] = __float2bfloat16_rn(lo);
    dst[f_hi - f_lo] = __float2bfloat16_rn(hi);
  }
}

template <int MT, int NT>
int launch_skinny(const void* x, int ldx, const void* w, void* y, int ldy, int M, int N, int K, int mode,
                  float out_scale, int n_split, long long split_stride, const void* ahead, long long ahead_bytes,
                  cudaStream_t stream) {
  const int feats = mode == SK_OUT_SWIGLU ? N / 2 : N;
  const int per_block = mode == SK_OUT_SWIGLU ? MT * 8 : MT * 16;
  dim3 grid((feats + per_block - 1) / per_block, n_split);
  const size_t smem = static_cast<size_t>(SK_WARPS) * MT * 16 * NT * 8 * sizeof(float);
  static bool configured = false;
  if (smem > 48 * 1024 && !configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<MT, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  return launch_streaming(gemm_skinny_kernel<MT, NT>, grid, dim3(SK_THREADS), smem, stream, static_cast<const bf16*>(x), ldx,
                static_cast<const bf16*>(w), y, ldy, M, N, K, mode, out_scale, split_stride,
                pdl_mode() >= 1 ? ahead : nullptr, pdl_mode() >= 1 ? ahead_bytes : 0ll);
}

}  // namespace dl

// x: bf16 [M, K] rows of ldx elements (16-byte aligned rows), w: bf16 [N, K] contiguous, K a multiple of 8,
// M <= 64. mode 0: y bf16 [M, N]; mode 1: y fp32, n_split partial results of [M, ldy] floats each,
// split_stride floats apart; mode 2: w = [gate; up] (N even), y bf16 [M, N / 2] = silu(x Wg^T) * (x Wu^T).
// mode 3: nothing but the place of each row's largest output leaves the kernel: y = float [M][blocks] then
// int [M][blocks] (blocks = ceil(N / features per block), see dl_gemm_skinny_argmax_blocks), the largest value of every
// block's features and its feature index (the lowest among equals); out_scale must be positive.
// n_split > 1 needs mode 1. ahead, ahead_bytes: memory that the kernel after this one will stream (weights),
// requested into L2 before this kernel waits for the one in front of it; null / 0: nothing.
DL_EXPORT int dl_gemm_skinny(const void* x, int ldx, const void* w, void* y, int ldy, int M, int N, int K, int mode,
                             float out_scale, int n_split, long long split_stride, const void* ahead,
                             long long ahead_bytes, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || (K & 7) || (ldx & 7) || n_split < 1 || n_split > 64 || (n_split > 1 && mode != dl::SK_OUT_F32) ||
      (mode == dl::SK_OUT_SWIGLU && (N & 1)) || mode < 0 || mode > 3 || (mode == dl::SK_OUT_ARGMAX && !(out_scale > 0.0f)))
    return DL_ERR_UNSUPPORTED;
  if (M <= 8) return dl::launch_skinny<1, 1>(x, ldx, w, y, ldy, M, N, K, mode, out_scale, n_split, split_stride, ahead, ahead_bytes, stream);
  if (M <= 16) return dl::launch_skinny<1, 2>(x, ldx, w, y, ldy, M, N, K, mode, out_scale, n_split, split_stride, ahead, ahead_bytes, stream);
  if (M <= 32) return dl::launch_skinny<2, 4>(x, ldx, w, y, ldy, M, N, K, mode, out_scale, n_split, split_stride, ahead, ahead_bytes, stream);
  return dl::launch_skinny<2, 8>(x, ldx, w, y, ldy, M, N, K, mode, out_scale, n_split, split_stride, ahead, ahead_bytes, stream);
}

// Blocks (= partial results per row) of dl_gemm_skinny in mode 3 for M rows and N features.
DL_EXPORT int dl_gemm_skinny_argmax_blocks(int M, int N) {
  const int per_block = M <= 16 ? 16 : 32;
  return (N + per_block - 1) / per_block;
}

// The fused q | k | v projection (see gemm_skinny_qkv_rope_kernel): x bf16 [M, K], M <= 16; w bf16 [(n_heads +
// 2 n_kv_heads) * head_dim, K]; q_out bf16 [M, ldq]; caches [pages, page_size, n_kv_heads, head_dim]; the whole
// head is rotated (rotary width = head_dim), head_dim a multiple of 16.
DL_EXPORT int dl_gemm_skinny_qkv_rope(const void* x, int ldx, const void* w, void* q_out, int ldq, int M, int K,
                                      const int* positions, const int* row_request, const int* block_table, int max_blocks,
                                      void* k_cache, void* v_cache, const float* inv_freq, float pos_scale, int n_heads,
                                      int n_kv_heads, int head_dim, int page_size, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (M > 16 || K <= 0 || (K & 7) || (ldx & 7) || head_dim <= 0 || (head_dim & 15) || n_heads <= 0 || n_kv_heads <= 0 ||
      page_size <= 0 || inv_freq == nullptr)
    return DL_ERR_UNSUPPORTED;
  dl::QkvRope p;
  p.positions = positions;
  p.row_request = row_request;
  p.block_table = block_table;
  p.max_blocks = max_blocks;
  p.k_cache = static_cast<dl::bf16*>(k_cache);
  p.v_cache = static_cast<dl::bf16*>(v_cache);
  p.inv_freq = inv_freq;
  p.angles = nullptr;
  p.pos_scale = pos_scale;
  p.n_heads = n_heads;
  p.n_kv_heads = n_kv_heads;
  p.head_dim = head_dim;
  p.page_size = page_size;
  const dim3 grid((n_heads + 2 * n_kv_heads) * (head_dim / 16));
  if (M <= 8) {
    const size_t smem = static_cast<size_t>(dl::SK_WARPS) * 16 * 8 * sizeof(float);
    return dl::launch_streaming(dl::gemm_skinny_qkv_rope_kernel<1>, grid, dim3(dl::SK_THREADS), smem, stream,
                      static_cast<const dl::bf16*>(x), ldx, static_cast<const dl::bf16*>(w), static_cast<dl::bf16*>(q_out), ldq,
                      M, K, p);
  }
  const size_t smem = static_cast<size_t>(dl::SK_WARPS) * 16 * 16 * sizeof(float);
  return dl::launch_streaming(dl::gemm_skinny_qkv_rope_kernel<2>, grid, dim3(dl::SK_THREADS), smem, stream,
                    static_cast<const dl::bf16*>(x), ldx, static_cast<const dl::bf16*>(w), static_cast<dl::bf16*>(q_out), ldq,
                    M, K, p);
}
