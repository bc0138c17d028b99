// y = x W^T on the 5th-generation tensor cores: tcgen05.mma with the accumulator in tensor memory,
// operands brought to shared memory by TMA. bf16 operands, fp32 accumulation.
//
// One thread block computes a 128 x BN tile of y (BN = 256, or 2 x 128 for SwiGLU). Roles:
//   warp 0, one lane   TMA producer: for each 64-wide slice of K, waits for a free stage, arms the stage's
//                      mbarrier with the byte count and issues the tile loads (x: 128 rows, W: BN rows), both
//                      K-major with the 128-byte swizzle that the tensor core reads directly
//   warp 1, one lane   issues four tcgen05.mma (M 128, N BN, K 16) per stage into the TMEM accumulator and
//                      commits them to the stage's "empty" barrier; after the last slice commits to the
//                      "accumulator ready" barrier. Warp 1 also allocates and frees the TMEM columns.
//   warps 2..5         epilogue: each warp reads its quarter of the 128 TMEM lanes (one output row per thread),
//                      converts and stores: bf16, fp32 (optionally scaled), or SwiGLU, where the tile's first
//                      128 columns are gate features and the last 128 the matching up features of W = [Wg; Wu].
// Rows, columns and K past the ends are zero-filled by TMA on the way in and masked on the way out.
//
// Every wait on an mbarrier is bounded: after about a second without progress the waiting role records a code
// in *status, and all roles fall through to the common exit, where the TMEM columns are freed. A block never
// spins forever and never leaves tensor memory allocated.
//
// The reference reaches its GPU matrix products through a library (ggml_mul_mat,
// dynacore/src/gpu/ggml_graph.cpp:278-292) and fuses the gated activation only on its CPU path
// (matmul_gated, dynacore/include/dynacore/device/device.h:188-199).
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace dl {

constexpr int T5_BM = 128;
constexpr int T5_BN = 256;
constexpr int T5_BK = 64;                 // 64 bf16 = 128 bytes: one swizzle row
constexpr int T5_STAGES = 4;
constexpr int T5_THREADS = 192;           // 6 warps
constexpr uint32_t T5_A_BYTES = T5_BM * T5_BK * 2;    // 16 KiB
constexpr uint32_t T5_B_BYTES = T5_BN * T5_BK * 2;    // 32 KiB
constexpr uint32_t T5_STAGE_BYTES = T5_A_BYTES + T5_B_BYTES;
constexpr uint32_t T5_TMEM_COLS = 256;
constexpr size_t T5_SMEM = static_cast<size_t>(T5_STAGES) * T5_STAGE_BYTES + 1024 /* alignment */ + 256 /* barriers */;

enum { T5_OUT_BF16 = 0, T5_OUT_F32 = 1, T5_OUT_SWIGLU = 2 };
enum { T5_ERR_PRODUCER = 1, T5_ERR_MMA = 2, T5_ERR_EPILOGUE = 3 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity. False (and *status set) after about a second.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code) {
  const uint32_t addr = smem_u32(bar);
  const long long start = clock64();
  for (uint32_t spins = 0;; ++spins) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
    if ((spins & 1023u) == 1023u && clock64() - start > 2000000000ll) {
      atomicExch(status, code);
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor for a K-major tile with 128-byte rows and 128-byte swizzle:
// start address >> 4 | stride between 8-row groups (1024 B) >> 4 at bit 32 | version 1 at bit 46 | swizzle 128B (2) at bit 61.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(1) << 16) |
         (static_cast<uint64_t>(1024 >> 4) << 32) | (static_cast<uint64_t>(1) << 46) | (static_cast<uint64_t>(2) << 61);
}

// Instruction descriptor: D fp32 (1 at bit 4), A and B bf16 (1 at bits 7 and 10), both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

// gate_rows: for SwiGLU the number of gate features F (W has 2F rows); the tile's W rows are
// [n0, n0 + 128) and [F + n0, F + n0 + 128). Otherwise unused.
__global__ void __launch_bounds__(T5_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    void* __restrict__ y, int ldy, int M, int N, int K, int mode, float out_scale, int gate_rows,
                    int* __restrict__ status) {
  extern __shared__ unsigned char t5_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(t5_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + static_cast<size_t>(T5_STAGES) * T5_STAGE_BYTES);
  uint64_t* full_bar = bars;                        // [T5_STAGES]
  uint64_t* empty_bar = bars + T5_STAGES;           // [T5_STAGES]
  uint64_t* acc_bar = bars + 2 * T5_STAGES;         // accumulator ready
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * T5_STAGES + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool swiglu = mode == T5_OUT_SWIGLU;
  const int n_per_tile = swiglu ? T5_BN / 2 : T5_BN;      // output features per tile
  const int n0 = blockIdx.x * n_per_tile, m0 = blockIdx.y * T5_BM;
  const int k_tiles = (K + T5_BK - 1) / T5_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T5_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_bar, 1);
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

  if (warp == 0) {
    if (lane == 0) {
      for (int kt = 0; kt < k_tiles; ++kt) {
        const int s = kt % T5_STAGES;
        if (kt >= T5_STAGES && !mbar_wait(&empty_bar[s], ((kt / T5_STAGES) & 1) ^ 1, status, T5_ERR_PRODUCER)) break;
        unsigned char* a_dst = tiles + static_cast<size_t>(s) * T5_STAGE_BYTES;
        unsigned char* b_dst = a_dst + T5_A_BYTES;
        mbar_expect_tx(&full_bar[s], T5_STAGE_BYTES);
        tma_load_2d(a_dst, &map_x, kt * T5_BK, m0, &full_bar[s]);
        if (swiglu) {
          tma_load_2d(b_dst, &map_w, kt * T5_BK, n0, &full_bar[s]);
          tma_load_2d(b_dst + T5_B_BYTES / 2, &map_w, kt * T5_BK, gate_rows + n0, &full_bar[s]);
        } else {
          tma_load_2d(b_dst, &map_w, kt * T5_BK, n0, &full_bar[s]);
          tma_load_2d(b_dst + T5_B_BYTES / 2, &map_w, kt * T5_BK, n0 + T5_BN / 2, &full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(T5_BM, T5_BN);
      bool ok = true;
      for (int kt = 0; kt < k_tiles && ok; ++kt) {
        const int s = kt % T5_STAGES;
        ok = mbar_wait(&full_bar[s], (kt / T5_STAGES) & 1, status, T5_ERR_MMA);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_u32(tiles + static_cast<size_t>(s) * T5_STAGE_BYTES);
        const uint32_t b_addr = a_addr + T5_A_BYTES;
#pragma unroll
        for (int k = 0; k < T5_BK / 16; ++k) {
          // 16 elements of K = 32 bytes further along the swizzled row
          umma_bf16(tmem_base, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(b_addr + k * 32), idesc,
                    (kt > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);      // arrives when these MMAs have finished reading the stage
      }
      umma_commit(acc_bar);              // arrives when every MMA issued so far has completed
    }
  } else {
    // epilogue: warp w may touch TMEM lanes 32 * (w % 4) .. + 31
    const int quarter = warp & 3;
    const int row = m0 + quarter * 32 + lane;
    // one lane polls; the whole warp then takes the same branch (tcgen05.ld is warp-wide)
    int ready = 0;
    if (lane == 0) ready = mbar_wait(acc_bar, 0, status, T5_ERR_EPILOGUE) ? 1 : 0;
    ready = __shfl_sync(0xffffffffu, ready, 0);
    if (ready) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      if (swiglu) {
        bf16* out = static_cast<bf16*>(y);
        for (int c = 0; c < T5_BN / 2; c += 32) {
          uint32_t g[32], u[32];
          tmem_ld32(lane_addr + c, g);
          tmem_ld32(lane_addr + T5_BN / 2 + c, u);
          if (row < M) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const int col = n0 + c + j;
              if (col < gate_rows) {           // gate_rows is a multiple of 8
                uint32_t w4[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float g0 = __uint_as_float(g[j + 2 * e]), g1 = __uint_as_float(g[j + 2 * e + 1]);
                  const float u0 = __uint_as_float(u[j + 2 * e]), u1 = __uint_as_float(u[j + 2 * e + 1]);
                  w4[e] = pack2_bf16(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
                }
                *reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * ldy + col) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
              }
            }
          }
        }
      } else {
        for (int c = 0; c < T5_BN; c += 32) {
          uint32_t v[32];
          tmem_ld32(lane_addr + c, v);
          if (row < M) {
            if (mode == T5_OUT_F32) {
              float* out = static_cast<float*>(y) + static_cast<size_t>(row) * ldy;
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                const int col = n0 + c + j;
                if (col < N)                    // N is a multiple of 4 in this mode
                  *reinterpret_cast<float4*>(out + col) =
                      make_float4(__uint_as_float(v[j]) * out_scale, __uint_as_float(v[j + 1]) * out_scale,
                                  __uint_as_float(v[j + 2]) * out_scale, __uint_as_float(v[j + 3]) * out_scale);
              }
            } else {
              bf16* out = static_cast<bf16*>(y) + static_cast<size_t>(row) * ldy;
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                const int col = n0 + c + j;
                if (col < N)                    // N is a multiple of 8 in this mode
                  *reinterpret_cast<uint4*>(out + col) = make_uint4(
                      pack2_bf16(__uint_as_float(v[j]) * out_scale, __uint_as_float(v[j + 1]) * out_scale),
                      pack2_bf16(__uint_as_float(v[j + 2]) * out_scale, __uint_as_float(v[j + 3]) * out_scale),
                      pack2_bf16(__uint_as_float(v[j + 4]) * out_scale, __uint_as_float(v[j + 5]) * out_scale),
                      pack2_bf16(__uint_as_float(v[j + 6]) * out_scale, __uint_as_float(v[j + 7]) * out_scale));
              }
            }
          }
        }
      }
    }
  }
  // common exit: every role arrives here, with or without a timeout
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(T5_TMEM_COLS) : "memory");
  }
}

// ---- host side -------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// rows x cols bf16, row pitch `ld` elements, box = box_rows x 64 columns, 128-byte swizzle, zero fill outside.
static int make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
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
DL_EXPORT int dl_gemm_tcgen05(const void* x, int ldx, const void* w, void* y, int ldy, int M, int N, int K, int mode,
                              float out_scale, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || (ldx & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      status == nullptr || mode < 0 || mode > 2)
    return DL_ERR_UNSUPPORTED;
  const int feats = mode == dl::T5_OUT_SWIGLU ? N / 2 : N;
  if ((mode == dl::T5_OUT_SWIGLU && (N & 1)) || (mode == dl::T5_OUT_F32 ? (feats & 3) || (ldy & 3) : (feats & 7) || (ldy & 7)) ||
      (reinterpret_cast<uintptr_t>(y) & 15))
    return DL_ERR_UNSUPPORTED;
  CUtensorMap map_x, map_w;
  int rc = dl::make_map(&map_x, x, M, K, ldx, dl::T5_BM);
  if (rc != 0) return rc;
  rc = dl::make_map(&map_w, w, N, K, K, dl::T5_BN / 2);
  if (rc != 0) return rc;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(dl::gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(dl::T5_SMEM));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const int per_tile = mode == dl::T5_OUT_SWIGLU ? dl::T5_BN / 2 : dl::T5_BN;
  dim3 grid((feats + per_tile - 1) / per_tile, (M + dl::T5_BM - 1) / dl::T5_BM);
  if (grid.y > 65535) return DL_ERR_UNSUPPORTED;
  dl::gemm_tcgen05_kernel<<<grid, dl::T5_THREADS, dl::T5_SMEM, stream>>>(map_x, map_w, y, ldy, M, N, K, mode, out_scale,
                                                                        mode == dl::T5_OUT_SWIGLU ? N / 2 : 0, status);
  return dl::launch_status();
}
