// y = x W^T for up to 64 rows on the 5th-generation tensor cores, built around the stream of W from HBM.
//
// The product is computed transposed, y^T = W x^T: 128 rows of W (output features) are the M side of a
// tcgen05.mma, the batch rows of x its N side (NB = 16, 32 or 64 columns of tensor memory), so a thread block
// streams a [128, K] piece of W once through a deep TMA pipeline (8 to 10 stages of 16 KiB) while x, a few KiB per
// k-slice, comes along from L2. One block per (feature tile, K split); K is split when there are too few feature
// tiles to occupy the GPU, and the splits then leave fp32 partial sums for the consumer to add in a fixed order
// (the residual-add + RMSNorm kernel does). Roles: warp 0 TMA producer, warp 1 MMA issue and tensor-memory
// allocation, warps 2..5 epilogue (thread = feature, NB batch values each).
//
// Epilogues: bf16 or fp32 store (transposed back to [rows, features]; 32 lanes write 32 consecutive features of
// one row), fp32 partial sums, and SwiGLU (a tile holds 64 gate features and the 64 matching up features of W =
// [Wg; Wu]; the halves meet through shared memory).
//
// The kernel starts before the kernel in front of it has ended (programmatic dependent launch): W does not depend
// on that kernel, so the first stages of W are requested at once; x and all stores wait.
//
// Every wait on an mbarrier is bounded (tcgen05.cuh); on a timeout all roles fall through to the common exit,
// where tensor memory is freed, and *status tells the host.
//
// The reference reaches its GPU matrix products through a library (ggml_mul_mat,
// dynacore/src/gpu/ggml_graph.cpp:278-292) and fuses the gated activation only on its CPU path (matmul_gated,
// dynacore/include/dynacore/device/device.h:188-199).
#include "common.cuh"
#include "tcgen05.cuh"

namespace dl {

constexpr int GS_BM = 128;                 // features per tile
constexpr int GS_BK = 64;                  // 64 bf16 = 128 bytes: one swizzle row
constexpr int GS_THREADS = 192;
constexpr uint32_t GS_A_BYTES = GS_BM * GS_BK * 2;
enum { GS_OUT_BF16 = 0, GS_OUT_F32 = 1, GS_OUT_SWIGLU = 2 };
enum { GS_ERR_PRODUCER = 21, GS_ERR_MMA = 22, GS_ERR_EPILOGUE = 23 };

template <int NB> struct GS {
  static constexpr int STAGES = NB <= 32 ? 10 : 8;
  static constexpr uint32_t B_BYTES = NB * GS_BK * 2;
  static constexpr uint32_t STAGE_BYTES = GS_A_BYTES + (B_BYTES < 1024 ? 1024 : B_BYTES);    // stages stay 1024-byte aligned
  static constexpr uint32_t TMEM_COLS = NB < 32 ? 32 : NB;
  static constexpr size_t SMEM = static_cast<size_t>(STAGES) * STAGE_BYTES + 1024 /* alignment */ + 256 /* barriers */;
};

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

// The four epilogue warps meet (named barrier 1, 128 threads).
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// gate_rows: for SwiGLU the number of gate features F (W has 2F rows); the tile's W rows are [j0, j0 + 64) and
// [F + j0, F + j0 + 64), j0 = 64 * blockIdx.x. split_stride: floats between the partial results of two K splits.
template <int NB>
__global__ void __launch_bounds__(GS_THREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, void* __restrict__ y,
                   int ldy, int M, int N, int K, int mode, float out_scale, int gate_rows, long long split_stride,
                   int* __restrict__ status) {
  constexpr int STAGES = GS<NB>::STAGES;
  constexpr uint32_t STAGE_BYTES = GS<NB>::STAGE_BYTES, B_BYTES = GS<NB>::B_BYTES, TMEM_COLS = GS<NB>::TMEM_COLS;
  extern __shared__ unsigned char gs_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gs_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + static_cast<size_t>(STAGES) * STAGE_BYTES);
  uint64_t* full_bar = bars;                 // [STAGES]
  uint64_t* empty_bar = bars + STAGES;       // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* exchange = reinterpret_cast<float*>(tiles);      // [NB][64] floats, over the stages once every MMA has read them

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool swiglu = mode == GS_OUT_SWIGLU;
  const int f0 = blockIdx.x * (swiglu ? GS_BM / 2 : GS_BM);        // first output feature (SwiGLU: first gate feature)
  const int n_split = gridDim.y, split = blockIdx.y;
  const int k_slices = (K + GS_BK - 1) / GS_BK;
  const int per = (k_slices + n_split - 1) / n_split;
  const int kt_begin = split * per, kt_end = min(k_slices, kt_begin + per);
  const int n_kt = max(0, kt_end - kt_begin);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_before_sync();
  __syncthreads();
  tcgen05_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // W first: it does not depend on the kernel before this one
    auto load_w = [&](int i) {
      const int s = i % STAGES;
      unsigned char* a_dst = tiles + static_cast<size_t>(s) * STAGE_BYTES;
      mbar_expect_tx(&full_bar[s], GS_A_BYTES + B_BYTES);
      if (swiglu) {
        tma_load_2d(a_dst, &map_w, (kt_begin + i) * GS_BK, f0, &full_bar[s]);
        tma_load_2d(a_dst + GS_A_BYTES / 2, &map_w, (kt_begin + i) * GS_BK, gate_rows + f0, &full_bar[s]);
      } else {
        tma_load_2d(a_dst, &map_w, (kt_begin + i) * GS_BK, f0, &full_bar[s]);
        tma_load_2d(a_dst + GS_A_BYTES / 2, &map_w, (kt_begin + i) * GS_BK, f0 + GS_BM / 2, &full_bar[s]);
      }
    };
    auto load_x = [&](int i) {
      const int s = i % STAGES;
      tma_load_2d(tiles + static_cast<size_t>(s) * STAGE_BYTES + GS_A_BYTES, &map_x, (kt_begin + i) * GS_BK, 0, &full_bar[s]);
    };
    const int ahead = min(n_kt, STAGES);
    if (elect_one())
      for (int i = 0; i < ahead; ++i) load_w(i);
    __syncwarp();
    pdl_wait();
    pdl_trigger();
    if (elect_one())
      for (int i = 0; i < ahead; ++i) load_x(i);
    __syncwarp();
    for (int i = ahead; i < n_kt; ++i) {
      if (!warp_wait(&empty_bar[i % STAGES], ((i / STAGES) & 1) ^ 1, status, GS_ERR_PRODUCER, abort_flag)) break;
      if (elect_one()) {
        load_w(i);
        load_x(i);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    pdl_wait();
    pdl_trigger();
    constexpr uint32_t idesc = umma_idesc(GS_BM, NB);
    const uint64_t desc0 = umma_desc_sw128(smem_u32(tiles));
    bool ok = true;
    for (int i = 0; i < n_kt; ++i) {
      const int s = i % STAGES;
      if (!warp_wait(&full_bar[s], (i / STAGES) & 1, status, GS_ERR_MMA, abort_flag)) {
        ok = false;
        break;
      }
      tcgen05_after_sync();
      if (elect_one()) {
        const uint64_t a_desc = desc0 + ((static_cast<uint32_t>(s) * STAGE_BYTES) >> 4);
        const uint64_t b_desc = a_desc + (GS_A_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < GS_BK / 16; ++k) umma_bf16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      __syncwarp();
    }
    if (ok && n_kt > 0 && elect_one()) umma_commit(acc_full);
    __syncwarp();
  } else {
    pdl_wait();
    pdl_trigger();
    // thread = feature: tensor-memory lane 32 * (warp % 4) + lane
    const int quarter = warp & 3;
    const int fl = quarter * 32 + lane;                  // feature inside the tile
    if (n_kt == 0 && mode == GS_OUT_F32 && f0 + fl < N) {
      // a K split that got no slice still owes its partial sums: zeros
      float* out = static_cast<float*>(y) + static_cast<size_t>(split) * split_stride + f0 + fl;
      for (int b = 0; b < M; ++b) out[static_cast<size_t>(b) * ldy] = 0.0f;
    }
    const bool ready = n_kt > 0 && warp_wait(acc_full, 0, status, GS_ERR_EPILOGUE, abort_flag);
    if (ready) {
      float acc[NB];
      tcgen05_after_sync();
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll
      for (int c0 = 0; c0 < NB; c0 += 16) {
        uint32_t v[16];
        tmem_ld16(lane_addr + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[c0 + j] = __uint_as_float(v[j]);
      }
      if (mode == GS_OUT_BF16 || mode == GS_OUT_F32) {
        const int f = f0 + fl;
        if (f < N) {
          if (mode == GS_OUT_F32) {
            float* out = static_cast<float*>(y) + static_cast<size_t>(split) * split_stride + f;
#pragma unroll
            for (int b = 0; b < NB; ++b)
              if (b < M) out[static_cast<size_t>(b) * ldy] = acc[b] * out_scale;
          } else {
            bf16* out = static_cast<bf16*>(y) + f;
#pragma unroll
            for (int b = 0; b < NB; ++b)
              if (b < M) out[static_cast<size_t>(b) * ldy] = __float2bfloat16_rn(acc[b] * out_scale);
          }
        }
      } else if (mode == GS_OUT_SWIGLU) {
        // lanes 0..63 hold gate features f0 + fl, lanes 64..127 the matching up features. The two halves swap half of
        // their batch columns through shared memory (every MMA has completed, so the stages are free): a gate thread
        // finishes columns [0, NB / 2) of its feature, the up thread of the same feature columns [NB / 2, NB).
        const bool is_gate = fl < 64;
        const int feat = is_gate ? fl : fl - 64;
        constexpr int HALF = NB / 2;
#pragma unroll
        for (int b = 0; b < HALF; ++b) {
          // what the partner needs: the gate thread's late columns, the up thread's early columns
          exchange[(is_gate ? HALF + b : b) * 64 + feat] = is_gate ? acc[HALF + b] : acc[b];
        }
        epilogue_sync();
        if (f0 + feat < gate_rows) {
          bf16* out = static_cast<bf16*>(y) + f0 + feat;
#pragma unroll
          for (int b = 0; b < HALF; ++b) {
            const int col = is_gate ? b : HALF + b;
            if (col < M) {
              const float other = exchange[col * 64 + feat];
              const float g = is_gate ? acc[b] : other, u = is_gate ? other : acc[HALF + b];
              out[static_cast<size_t>(col) * ldy] = __float2bfloat16_rn(__fdividef(g, 1.0f + __expf(-g)) * u);
            }
          }
        }
      }
    }
  }
  // common exit: every role arrives here, with or without a timeout
  drain_after_abort(abort_flag);
  tcgen05_before_sync();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// rows x cols bf16 with a row pitch of `ld` elements; box = box_rows x 64 columns, 128-byte swizzle, zero fill outside.
static int gs_make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  EncodeTiledFn fn = tensor_map_encoder();
  if (fn == nullptr) return DL_ERR_UNSUPPORTED;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(GS_BK), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 700000 + static_cast<int>(r);
}

template <int NB>
static int gs_launch(const CUtensorMap& map_w, const CUtensorMap& map_x, void* y, int ldy, int M, int N, int K, int mode,
                     float out_scale, int gate_rows, int n_tiles, int n_split, long long split_stride, int* status,
                     cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(GS<NB>::SMEM));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  return launch_streaming(gemm_stream_kernel<NB>, dim3(n_tiles, n_split), dim3(GS_THREADS), GS<NB>::SMEM, stream, map_w, map_x,
                          y, ldy, M, N, K, mode, out_scale, gate_rows, split_stride, status);
}

static int gs_run(const void* x, int ldx, const void* w, void* y, int ldy, int M, int N, int K, int mode, float out_scale,
                  int n_split, long long split_stride, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || (K & 7) || (ldx & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      status == nullptr || n_split < 1 || n_split > 64 || (n_split > 1 && mode != GS_OUT_F32) ||
      (mode == GS_OUT_SWIGLU && (N & 1)))
    return DL_ERR_UNSUPPORTED;
  const int gate_rows = mode == GS_OUT_SWIGLU ? N / 2 : 0;
  const int feats = mode == GS_OUT_SWIGLU ? N / 2 : N;
  const int per_tile = mode == GS_OUT_SWIGLU ? GS_BM / 2 : GS_BM;
  const int n_tiles = (feats + per_tile - 1) / per_tile;
  CUtensorMap map_w, map_x;
  int rc = gs_make_map(&map_w, w, N, K, K, GS_BM / 2);
  if (rc != 0) return rc;
  const int nb = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  rc = gs_make_map(&map_x, x, M, K, ldx, nb);
  if (rc != 0) return rc;
  if (nb == 16)
    return gs_launch<16>(map_w, map_x, y, ldy, M, N, K, mode, out_scale, gate_rows, n_tiles, n_split, split_stride, status, stream);
  if (nb == 32)
    return gs_launch<32>(map_w, map_x, y, ldy, M, N, K, mode, out_scale, gate_rows, n_tiles, n_split, split_stride, status, stream);
  return gs_launch<64>(map_w, map_x, y, ldy, M, N, K, mode, out_scale, gate_rows, n_tiles, n_split, split_stride, status, stream);
}

}  // namespace dl

// x: bf16 [M, K] (M <= 64) rows of ldx elements; w: bf16 [N, K] contiguous; both 16-byte aligned, K and ldx multiples
// of 8. mode 0: y bf16 [M, N]; mode 1: y fp32, n_split partial results of [M, ldy] floats each, split_stride floats
// apart (n_split > 1 needs this mode); mode 2: w = [gate; up] with N = 2F rows, y bf16 [M, F] = silu(x Wg^T) * (x Wu^T).
// status: one device int, set to a nonzero code if a wait inside the kernel timed out (left untouched otherwise).
DL_EXPORT int dl_gemm_stream(const void* x, int ldx, const void* w, void* y, int ldy, int M, int N, int K, int mode,
                             float out_scale, int n_split, long long split_stride, int* status, cudaStream_t stream) {
  if (mode < 0 || mode > 2) return DL_ERR_UNSUPPORTED;
  return dl::gs_run(x, ldx, w, y, ldy, M, N, K, mode, out_scale, n_split, split_stride, status, stream);
}
