// The tcgen05 matrix product, shared by gemm_tcgen05.cu (every block for itself) and the cluster variant (two blocks
// share each W tile): the kernel, templated on how a block gets its operands, and its host-side launcher.
#pragma once

#include "qkv_rope.cuh"
#include "tcgen05.cuh"

namespace dl {

constexpr int T5_BM = 128;
constexpr int T5_BK = 64;                 // 64 bf16 = 128 bytes: one swizzle row
constexpr int T5_THREADS = 192;           // 6 warps
constexpr uint32_t T5_A_BYTES = T5_BM * T5_BK * 2;    // 16 KiB
constexpr uint32_t T5_STORE_BYTES = 4 * 32 * 128;     // per epilogue warp: 32 rows x 128 bytes of output, staged for coalesced stores

// Tile width BN is 256 (4 stages of 48 KiB), 192 (5 stages of 40 KiB) or 128 (6 stages of 32 KiB); the narrower
// ones are for shapes whose tile count fits the SMs badly at 256. SwiGLU takes 256 or 128 only.
template <int BN> struct T5 {
  static constexpr int STAGES = BN == 256 ? 4 : (BN == 192 ? 5 : 6);
  static constexpr uint32_t B_BYTES = BN * T5_BK * 2;
  static constexpr uint32_t STAGE_BYTES = T5_A_BYTES + B_BYTES;
  static constexpr uint32_t TMEM_COLS = BN == 128 ? 256 : 512;      // two accumulators (a power of two)
  static constexpr size_t SMEM = static_cast<size_t>(STAGES) * STAGE_BYTES + T5_STORE_BYTES + 1024 /* alignment */ + 256 /* barriers */;
};

enum { T5_OUT_BF16 = 0, T5_OUT_F32 = 1, T5_OUT_SWIGLU = 2, T5_OUT_QKV_ROPE = 3 };
enum { T5_ERR_PRODUCER = 1, T5_ERR_MMA = 2, T5_ERR_EPILOGUE = 3 };

// Which output tile a tile number stands for. Tiles are numbered in groups of `group_m` row blocks: inside a
// group the row block changes fastest, then the column block; the groups follow one another. The blocks of the grid
// work on consecutive numbers at any time, so together they hold group_m row blocks of x and gridDim.x / group_m
// column blocks of W: both stay in L2 while they are used, and over the whole product W comes from memory once
// per group and x once. (Numbered along the columns first, as this kernel did at first, every row block brings all
// of W in again: with the 235 MB of a 4096 -> 2 x 14336 gate|up matrix that bound the product to memory, 1,684 us
// for 8,192 rows where the arithmetic needs 1,300.)
__host__ __device__ __forceinline__ void t5_tile_coords(int tile, int tiles_n, int num_tiles, int group_m, int* m_tile, int* n_tile) {
  const int tiles_m = num_tiles / tiles_n;
  const int per_group = group_m * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * group_m;
  const int rows = group_m < tiles_m - first_m ? group_m : tiles_m - first_m;
  const int r = tile - g * per_group;
  *m_tile = first_m + r % rows;
  *n_tile = r / rows;
}

// gate_rows: for SwiGLU the number of gate features F (W has 2F rows); the tile's W rows are
// [n0, n0 + 128) and [F + n0, F + n0 + 128). Otherwise unused.
//
// The kernel is persistent: gridDim.x blocks (at most one per SM) walk the output tiles in the order
// tile = blockIdx.x, blockIdx.x + gridDim.x, ...; see t5_tile_coords for which tile a number stands for.
// The accumulator is double-buffered in tensor memory (2 x 256 columns): the epilogue warps drain
// one tile while the MMA warp fills the next.
//
// `P` says how a block gets its operands. P::CLUSTER == 1: every block loads both halves of its W tile itself.
// P::CLUSTER == 2: the two blocks of a thread-block cluster take row blocks 2i and 2i + 1 of the same column
// block; each loads one half of the shared W tile and its copy lands in both blocks' shared memory, so W crosses
// from L2 once per pair (measured: the kernel is bound by operand traffic from L2; loading a third less made it
// a fifth faster). A stage is then free only when both blocks' MMAs have read it: each block's commit arrives on
// the stage's barrier in both blocks, and the barrier counts two arrivals.
template <int T5_BN, class P>
__global__ void __launch_bounds__(T5_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    void* __restrict__ y, int ldy, int M, int N, int K, int mode, float out_scale, int gate_rows,
                    int tiles_n, int num_tiles, int group_m, int* __restrict__ status, const QkvRope rope) {
  constexpr int T5_STAGES = T5<T5_BN>::STAGES;
  constexpr uint32_t T5_B_BYTES = T5<T5_BN>::B_BYTES, T5_STAGE_BYTES = T5<T5_BN>::STAGE_BYTES, T5_TMEM_COLS = T5<T5_BN>::TMEM_COLS;
  extern __shared__ unsigned char t5_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(t5_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* store_stage = tiles + static_cast<size_t>(T5_STAGES) * T5_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(store_stage + T5_STORE_BYTES);
  uint64_t* full_bar = bars;                        // [T5_STAGES] stage loaded
  uint64_t* empty_bar = bars + T5_STAGES;           // [T5_STAGES] stage consumed
  uint64_t* acc_full = bars + 2 * T5_STAGES;        // [2] accumulator complete
  uint64_t* acc_empty = bars + 2 * T5_STAGES + 2;   // [2] accumulator drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * T5_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // in a cluster: this block's rank, and the walk over pairs of row blocks instead of single tiles
  const int rank = P::CLUSTER == 2 ? static_cast<int>(cluster_rank()) : 0;
  const int first_tile = P::CLUSTER == 2 ? static_cast<int>(blockIdx.x) / 2 : static_cast<int>(blockIdx.x);
  const int tile_step = P::CLUSTER == 2 ? static_cast<int>(gridDim.x) / 2 : static_cast<int>(gridDim.x);
  const bool swiglu = mode == T5_OUT_SWIGLU;
  const int n_per_tile = swiglu ? T5_BN / 2 : T5_BN;      // output features per tile
  const int k_tiles = (K + T5_BK - 1) / T5_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T5_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], P::CLUSTER);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);                  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(T5_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  if constexpr (P::CLUSTER == 2) cluster_sync_all();      // the partner's barriers exist before anything is sent to them

  if (warp == 0) {
    // TMA producer: the whole warp runs the loop (every lane polls the barrier), one elected lane issues the copies
    // The first stages' slices of W are requested before the wait on the kernel in front (programmatic dependent
    // launch): W does not depend on it. x, which does, follows after the wait.
    auto load_w = [&](int s, int kt, int n0) {
      unsigned char* b_dst = tiles + static_cast<size_t>(s) * T5_STAGE_BYTES + T5_A_BYTES;
      const int second_half = swiglu ? gate_rows + n0 : n0 + T5_BN / 2;      // W row of the tile's second half
      if constexpr (P::CLUSTER == 2) {
        // this block's half of the W tile, into both blocks (the partner sends the other half)
        P::load_shared_half(b_dst + rank * (T5_B_BYTES / 2), &map_w, kt * T5_BK, rank == 0 ? n0 : second_half, &full_bar[s]);
      } else {
        tma_load_2d(b_dst, &map_w, kt * T5_BK, n0, &full_bar[s]);
        tma_load_2d(b_dst + T5_B_BYTES / 2, &map_w, kt * T5_BK, second_half, &full_bar[s]);
      }
    };
    auto load_x = [&](int s, int kt, int m0) {
      tma_load_2d(tiles + static_cast<size_t>(s) * T5_STAGE_BYTES, &map_x, kt * T5_BK, m0, &full_bar[s]);
    };
    const int ahead = first_tile < num_tiles ? min(k_tiles, T5_STAGES) : 0;
    if (ahead > 0) {
      int m_tile, n_tile;
      t5_tile_coords(first_tile, tiles_n, num_tiles, group_m, &m_tile, &n_tile);
      const int m0 = (m_tile * P::CLUSTER + rank) * T5_BM, n0 = n_tile * n_per_tile;
      if (elect_one()) {
        for (int kt = 0; kt < ahead; ++kt) {
          mbar_expect_tx(&full_bar[kt], T5_STAGE_BYTES);
          load_w(kt, kt, n0);
        }
      }
      __syncwarp();
      pdl_wait();
      pdl_trigger();
      if (elect_one()) {
        for (int kt = 0; kt < ahead; ++kt) load_x(kt, kt, m0);
      }
      __syncwarp();
    } else {
      pdl_wait();
      pdl_trigger();
    }
    uint32_t it = ahead;                           // k-slices issued so far, over all tiles
    bool ok = true;
    for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
      int m_tile, n_tile;
      t5_tile_coords(tile, tiles_n, num_tiles, group_m, &m_tile, &n_tile);
      const int m0 = (m_tile * P::CLUSTER + rank) * T5_BM, n0 = n_tile * n_per_tile;
      for (int kt = tile == first_tile ? ahead : 0; kt < k_tiles; ++kt, ++it) {
        const int s = it % T5_STAGES;
        if (it >= T5_STAGES && !warp_wait(&empty_bar[s], ((it / T5_STAGES) & 1) ^ 1, status, T5_ERR_PRODUCER, abort_flag)) {
          ok = false;
          break;
        }
        if (elect_one()) {
          mbar_expect_tx(&full_bar[s], T5_STAGE_BYTES);
          load_x(s, kt, m0);
          load_w(s, kt, n0);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    pdl_wait();
    pdl_trigger();
    // MMA issue: the whole warp runs the loop, one elected lane issues the instructions
    constexpr uint32_t idesc = umma_idesc(T5_BM, T5_BN);
    const uint64_t desc0 = umma_desc_sw128(smem_u32(tiles));      // a step along the tiles adds (bytes >> 4)
    uint32_t it = 0, local = 0;                    // k-slices consumed; tiles done by this block
    bool ok = true;
    for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step, ++local) {
      const uint32_t buf = local & 1;
      // the epilogue must have drained this buffer (its previous use was tile local - 2)
      if (local >= 2 && !warp_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, status, T5_ERR_MMA, abort_flag)) break;
      tcgen05_after_sync();
      const uint32_t acc = tmem_base + buf * T5_BN;
      for (int kt = 0; kt < k_tiles; ++kt, ++it) {
        const int s = it % T5_STAGES;
        if (!warp_wait(&full_bar[s], (it / T5_STAGES) & 1, status, T5_ERR_MMA, abort_flag)) {
          ok = false;
          break;
        }
        tcgen05_after_sync();
        if (elect_one()) {
          const uint64_t a_desc = desc0 + ((static_cast<uint32_t>(s) * T5_STAGE_BYTES) >> 4);
          const uint64_t b_desc = a_desc + (T5_A_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < T5_BK / 16; ++k) {
            // 16 elements of K = 32 bytes further along the swizzled row
            umma_bf16(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kt > 0 || k > 0) ? 1u : 0u);
          }
          P::commit_stage_free(&empty_bar[s]);       // arrives (in both blocks of a pair) when these MMAs have read the stage
        }
        __syncwarp();
      }
      if (ok && elect_one()) umma_commit(&acc_full[buf]);    // arrives when every MMA issued so far has completed
      __syncwarp();
    }
  } else {
    pdl_wait();
    pdl_trigger();
    // epilogue: warp w may touch TMEM lanes 32 * (w % 4) .. + 31
    const int quarter = warp & 3;
    uint32_t local = 0;
    for (int tile = first_tile; tile < num_tiles; tile += tile_step, ++local) {
      const uint32_t buf = local & 1;
      int m_tile, n_tile;
      t5_tile_coords(tile, tiles_n, num_tiles, group_m, &m_tile, &n_tile);
      const int m0 = (m_tile * P::CLUSTER + rank) * T5_BM, n0 = n_tile * n_per_tile;
      const int row = m0 + quarter * 32 + lane;
      if (!warp_wait(&acc_full[buf], (local >> 1) & 1, status, T5_ERR_EPILOGUE, abort_flag)) break;
      tcgen05_after_sync();
      const uint32_t lane_addr = tmem_base + buf * T5_BN + (static_cast<uint32_t>(quarter * 32) << 16);
      unsigned char* my_stage = store_stage + (warp - 2) * (T5_STORE_BYTES / 4);
      const int row0 = m0 + quarter * 32;
      if (swiglu) {
        bf16* out = static_cast<bf16*>(y);
        for (int c0 = 0; c0 < T5_BN / 2; c0 += 64) {
          uint4 w[8];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t g[32], u[32];
            tmem_ld32(lane_addr + c0 + hh * 32, g);
            tmem_ld32(lane_addr + T5_BN / 2 + c0 + hh * 32, u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint32_t w4[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float g0 = __uint_as_float(g[j + 2 * e]), g1 = __uint_as_float(g[j + 2 * e + 1]);
                const float u0 = __uint_as_float(u[j + 2 * e]), u1 = __uint_as_float(u[j + 2 * e + 1]);
                w4[e] = pack2_bf16(__fdividef(g0, 1.0f + __expf(-g0)) * u0, __fdividef(g1, 1.0f + __expf(-g1)) * u1);
              }
              w[hh * 4 + j / 8] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            }
          }
          store_rows_bf16(w, my_stage, lane, out, ldy, row0, M, n0 + c0, gate_rows);   // gate_rows is a multiple of 8
        }
      } else if (mode == T5_OUT_QKV_ROPE) {
        // W = [Wq; Wk; Wv]: a tile holds whole heads (head_dim 64 or 128 divides the tile width). Thread = row:
        // the two members of rotary pair i of a head are columns i and i + head_dim / 2 of the same thread.
        const bool live = row < M;
        const int pos = live ? rope.positions[row] : 0;
        const size_t slot = live ? qkv_rope_slot(rope, row, pos) : 0;
        const float fpos = static_cast<float>(pos) * rope.pos_scale;
        const int hd = rope.head_dim;
        const float4* my_angles = rope.angles != nullptr && live
                                      ? reinterpret_cast<const float4*>(rope.angles + static_cast<size_t>(row) * (hd / 2))
                                      : nullptr;       // two (cos, sin) pairs per 16-byte load
        // A warp past the last row has nothing to read or write; a row past it inside a live warp is carried along
        // unrotated (its sines and cosines are not looked up or worked out).
        const bool warp_live = row - lane < M;
        for (int h0 = 0; warp_live && h0 < T5_BN && n0 + h0 < N; h0 += hd) {
          const int head = (n0 + h0) / hd;                // q heads, then k heads, then v heads
          const bool rotated = head < rope.n_heads + rope.n_kv_heads;
          bf16* dst = nullptr;
          if (live) {
            if (head < rope.n_heads) {
              dst = static_cast<bf16*>(y) + static_cast<size_t>(row) * ldy + static_cast<size_t>(head) * hd;
            } else if (slot != QKV_NO_SLOT) {
              const bool is_k = head < rope.n_heads + rope.n_kv_heads;
              const int kvh = head - rope.n_heads - (is_k ? 0 : rope.n_kv_heads);
              dst = (is_k ? rope.k_cache : rope.v_cache) + (slot * rope.n_kv_heads + kvh) * hd;
            }
          }
          for (int piece = 0; piece < hd / 64; ++piece) {     // 32 pairs at a time
            uint32_t lo[32], hi[32];
            tmem_ld32(lane_addr + h0 + piece * 32, lo);
            tmem_ld32(lane_addr + h0 + hd / 2 + piece * 32, hi);
            tmem_ld_wait();
            // (cos, sin) of the piece's 32 pairs, two pairs per float4: all requested before any is used
            float4 cs[16];
            if (rotated && live) {
              if (my_angles != nullptr) {
#pragma unroll
                for (int i = 0; i < 16; ++i) cs[i] = my_angles[piece * 16 + i];
              } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  sincosf(fpos * rope.inv_freq[piece * 32 + 2 * i], &cs[i].y, &cs[i].x);
                  sincosf(fpos * rope.inv_freq[piece * 32 + 2 * i + 1], &cs[i].w, &cs[i].z);
                }
              }
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) cs[i] = make_float4(1.0f, 0.0f, 1.0f, 0.0f);     // v heads: no rotation
            }
            uint4 wlo[4], whi[4];
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint32_t pl[4], ph[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float a0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(lo[j + 2 * e])));
                const float a1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(lo[j + 2 * e + 1])));
                const float b0 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(hi[j + 2 * e])));
                const float b1 = __bfloat162float(__float2bfloat16_rn(__uint_as_float(hi[j + 2 * e + 1])));
                const float4 t4 = cs[j / 2 + e];
                pl[e] = pack2_bf16(a0 * t4.x - b0 * t4.y, a1 * t4.z - b1 * t4.w);
                ph[e] = pack2_bf16(a0 * t4.y + b0 * t4.x, a1 * t4.w + b1 * t4.z);
              }
              wlo[j / 8] = make_uint4(pl[0], pl[1], pl[2], pl[3]);
              whi[j / 8] = make_uint4(ph[0], ph[1], ph[2], ph[3]);
            }
            store_rows_pieces(wlo, whi, my_stage, lane, dst, piece * 32, hd / 2 + piece * 32);
          }
        }
      } else {
        for (int c0 = 0; c0 < T5_BN; c0 += 64) {
          uint32_t va[32], vb[32];
          tmem_ld32(lane_addr + c0, va);
          tmem_ld32(lane_addr + c0 + 32, vb);
          tmem_ld_wait();
          if (mode == T5_OUT_F32) {
            if (row < M) {
              float* out = static_cast<float*>(y) + static_cast<size_t>(row) * ldy;
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) {
                const uint32_t* v = hh == 0 ? va : vb;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                  const int col = n0 + c0 + hh * 32 + j;
                  if (col < N)                    // N is a multiple of 4 in this mode
                    *reinterpret_cast<float4*>(out + col) =
                        make_float4(__uint_as_float(v[j]) * out_scale, __uint_as_float(v[j + 1]) * out_scale,
                                    __uint_as_float(v[j + 2]) * out_scale, __uint_as_float(v[j + 3]) * out_scale);
                }
              }
            }
          } else {
            uint4 w[8];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              const uint32_t* v = hh == 0 ? va : vb;
#pragma unroll
              for (int j = 0; j < 32; j += 8)
                w[hh * 4 + j / 8] = make_uint4(
                    pack2_bf16(__uint_as_float(v[j]) * out_scale, __uint_as_float(v[j + 1]) * out_scale),
                    pack2_bf16(__uint_as_float(v[j + 2]) * out_scale, __uint_as_float(v[j + 3]) * out_scale),
                    pack2_bf16(__uint_as_float(v[j + 4]) * out_scale, __uint_as_float(v[j + 5]) * out_scale),
                    pack2_bf16(__uint_as_float(v[j + 6]) * out_scale, __uint_as_float(v[j + 7]) * out_scale));
            }
            store_rows_bf16(w, my_stage, lane, static_cast<bf16*>(y), ldy, row0, M, n0 + c0, N);   // N is a multiple of 8
          }
        }
      }
      // this warp has read its part of the buffer: let the MMA warp reuse it
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
    }
  }
  // common exit: every role arrives here, with or without a timeout
  drain_after_abort(abort_flag);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if constexpr (P::CLUSTER == 2) cluster_sync_all();      // nobody leaves while its partner may still send to it
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(T5_TMEM_COLS) : "memory");
  }
}

// ---- host side -------------------------------------------------------------------------------------

// rows x cols bf16, row pitch `ld` elements, box = box_rows x 64 columns, 128-byte swizzle, zero fill outside.
static inline int make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  EncodeTiledFn fn = tensor_map_encoder();
  if (fn == nullptr) return DL_ERR_UNSUPPORTED;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(T5_BK), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 700000 + static_cast<int>(r);
}

}  // namespace dl

// x: bf16 [M, K] rows of ldx elements; w: bf16 [N, K] contiguous; both 16-byte aligned with K and ldx multiples of 8.
// mode 0: y bf16 [M, N] (N % 8 == 0); mode 1: y fp32 [M, N] (N % 4 == 0); mode 2: w = [gate; up] with N = 2F rows,
// y bf16 [M, F] = silu(x Wg^T) * (x Wu^T) (F % 8 == 0). status: one device int, set to a nonzero code if a wait
// inside the kernel timed out (left untouched otherwise).
template <class P>
static int t5_launch(const void* x, int ldx, const void* w, void* y, int ldy, int M, int N, int K, int mode, float out_scale,
                     int* status, const dl::QkvRope& rope, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || (ldx & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      status == nullptr || mode < 0 || mode > 3)
    return DL_ERR_UNSUPPORTED;
  const int feats = mode == dl::T5_OUT_SWIGLU ? N / 2 : N;
  if ((mode == dl::T5_OUT_SWIGLU && (N & 1)) || (mode == dl::T5_OUT_F32 ? (feats & 3) || (ldy & 3) : (feats & 7) || (ldy & 7)) ||
      (reinterpret_cast<uintptr_t>(y) & 15))
    return DL_ERR_UNSUPPORTED;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
  }
  const long long m_blocks = (M + dl::T5_BM - 1) / dl::T5_BM;
  const long long m_tiles = (m_blocks + P::CLUSTER - 1) / P::CLUSTER;      // pairs of row blocks in a cluster
  // Tile width: the one whose rounds over the SMs cost least, a round of 192- or 128-wide tiles taking about 0.78
  // or 0.7 of a round of 256-wide ones (measured). SwiGLU pairs gate and up columns in halves of 64: 256 or 128. The
  // q | k | v epilogue needs whole heads in a tile.
  const int units = sm_count / P::CLUSTER;                                  // blocks, or clusters of two
  auto cost = [&](int bn, double per_round) {
    const int per = mode == dl::T5_OUT_SWIGLU ? bn / 2 : bn;
    const long long t = m_tiles * ((feats + per - 1) / per);
    return static_cast<double>((t + units - 1) / units) * per_round;
  };
  static int forced = -1;      // DYNALM_GEMM_TILE=128|192|256 overrides the choice where the width is allowed (for measurements)
  if (forced < 0) { const char* e = getenv("DYNALM_GEMM_TILE"); forced = e ? atoi(e) : 0; }
  int bn = 256;
  double best = cost(256, 1.0);
  const bool can192 = mode != dl::T5_OUT_SWIGLU && (mode != dl::T5_OUT_QKV_ROPE || 192 % rope.head_dim == 0);
  if (can192 && cost(192, 0.78) < best) {
    bn = 192;
    best = cost(192, 0.78);
  }
  if (cost(128, 0.7) < best) bn = 128;
  if (forced == 128 || forced == 256 || (forced == 192 && can192)) bn = forced;
  const int per_tile = mode == dl::T5_OUT_SWIGLU ? bn / 2 : bn;
  const int tiles_n = (feats + per_tile - 1) / per_tile;
  const long long tiles = m_tiles * tiles_n;
  if (tiles > (1ll << 30)) return DL_ERR_UNSUPPORTED;
  CUtensorMap map_x, map_w;
  int rc = dl::make_map(&map_x, x, M, K, ldx, dl::T5_BM);
  if (rc != 0) return rc;
  rc = dl::make_map(&map_w, w, N, K, K, bn / 2);
  if (rc != 0) return rc;
  // Row blocks to a group of tiles (t5_tile_coords): as many as keep the group's rows of x within about 32 MB of L2,
  // 4 to 16. DYNALM_GEMM_GROUP_M overrides it (1: along the columns first).
  static int forced_group = -1;
  if (forced_group < 0) { const char* e = getenv("DYNALM_GEMM_GROUP_M"); forced_group = e ? atoi(e) : 0; }
  long long group = (32ll << 20) / (2ll * dl::T5_BM * P::CLUSTER * K);
  group = group < 4 ? 4 : (group > 16 ? 16 : group);
  if (forced_group > 0) group = forced_group;
  const int group_m = static_cast<int>(group < m_tiles ? group : m_tiles);
  const int blocks = static_cast<int>(tiles < units ? tiles : units) * P::CLUSTER;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(dl::T5_THREADS);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (P::CLUSTER > 1) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = P::CLUSTER;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  if (dl::pdl_mode() >= 1) {      // the kernel may start before the one in front has ended: it requests W before its wait
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  const int gate_rows = mode == dl::T5_OUT_SWIGLU ? N / 2 : 0;
  if (bn == 256) {
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(dl::gemm_tcgen05_kernel<256, P>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(dl::T5<256>::SMEM));
      if (e != cudaSuccess) return static_cast<int>(e);
      configured = true;
    }
    cfg.dynamicSmemBytes = dl::T5<256>::SMEM;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, dl::gemm_tcgen05_kernel<256, P>, map_x, map_w, y, ldy, M, N, K, mode,
                                               out_scale, gate_rows, tiles_n, static_cast<int>(tiles), group_m, status, rope));
  } else if (bn == 192) {
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(dl::gemm_tcgen05_kernel<192, P>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(dl::T5<192>::SMEM));
      if (e != cudaSuccess) return static_cast<int>(e);
      configured = true;
    }
    cfg.dynamicSmemBytes = dl::T5<192>::SMEM;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, dl::gemm_tcgen05_kernel<192, P>, map_x, map_w, y, ldy, M, N, K, mode,
                                               out_scale, gate_rows, tiles_n, static_cast<int>(tiles), group_m, status, rope));
  } else {
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(dl::gemm_tcgen05_kernel<128, P>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(dl::T5<128>::SMEM));
      if (e != cudaSuccess) return static_cast<int>(e);
      configured = true;
    }
    cfg.dynamicSmemBytes = dl::T5<128>::SMEM;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, dl::gemm_tcgen05_kernel<128, P>, map_x, map_w, y, ldy, M, N, K, mode,
                                               out_scale, gate_rows, tiles_n, static_cast<int>(tiles), group_m, status, rope));
  }
}

// Fills the epilogue's parameters for the q | k | v product and launches it (see dl_gemm_tcgen05_qkv_rope).
template <class P>
static int t5_launch_qkv_rope(const void* x, int ldx, const void* w, void* q_out, int ldq, int M, int K, const int* positions,
                              const int* row_request, const int* block_table, int max_blocks, void* k_cache, void* v_cache,
                              const float* inv_freq, const void* angles, float pos_scale, int n_heads, int n_kv_heads,
                              int head_dim, int page_size, int* status, cudaStream_t stream) {
  if ((head_dim != 64 && head_dim != 128) || n_heads <= 0 || n_kv_heads <= 0 || page_size <= 0 || inv_freq == nullptr ||
      (reinterpret_cast<uintptr_t>(k_cache) & 15) || (reinterpret_cast<uintptr_t>(v_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(angles) & 15))
    return DL_ERR_UNSUPPORTED;
  dl::QkvRope p;
  p.positions = positions;
  p.row_request = row_request;
  p.block_table = block_table;
  p.max_blocks = max_blocks;
  p.k_cache = static_cast<dl::bf16*>(k_cache);
  p.v_cache = static_cast<dl::bf16*>(v_cache);
  p.inv_freq = inv_freq;
  p.angles = static_cast<const float2*>(angles);
  p.pos_scale = pos_scale;
  p.n_heads = n_heads;
  p.n_kv_heads = n_kv_heads;
  p.head_dim = head_dim;
  p.page_size = page_size;
  return t5_launch<P>(x, ldx, w, q_out, ldq, M, (n_heads + 2 * n_kv_heads) * head_dim, K, dl::T5_OUT_QKV_ROPE, 1.0f, status, p,
                      stream);
}
