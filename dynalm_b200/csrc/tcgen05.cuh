// tcgen05 / TMA / mbarrier building blocks shared by the kernels that run on the 5th-generation tensor
// cores (sm_100a): bounded mbarrier waits, tiled TMA loads, shared-memory matrix descriptors, the MMA
// itself, and tensor-memory loads and stores.
//
// Every wait is bounded: after about a second without progress the waiting role records a code in
// *status and raises the block's abort flag; all roles then fall through to the block's common exit,
// where tensor memory is freed. A block never spins forever and never leaves tensor memory allocated.
#pragma once

#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace dl {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity. False after about a second (then *status and the
// block's abort flag are set), or as soon as another role of the block has given up.
__device__ __forceinline__ bool mbar_try(uint32_t addr, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(addr), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code, volatile int* abort_flag) {
  const uint32_t addr = smem_u32(bar);
  if (mbar_try(addr, parity)) return true;      // the common case costs one instruction, no clock read
  long long start = 0;
  for (uint32_t spins = 1;; ++spins) {
    if (mbar_try(addr, parity)) return true;
    if ((spins & 255u) == 0u) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (start == 0) {
        start = now;
      } else if (now - start > 2000000000ll) {
        atomicExch(status, code);
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// Every lane polls (measured: a third of the cost of one polling lane followed by a broadcast); the vote makes the
// whole warp take the same branch, as the warp-wide tensor-memory instructions that follow need.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, int* status, int code, volatile int* abort_flag) {
  const bool ok = mbar_wait(bar, parity, status, code, abort_flag);
  return __all_sync(0xffffffffu, ok);
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
// True in exactly one lane of a converged warp, the same lane every time. The tensor-core and TMA instructions
// take their descriptors from uniform registers: issued from warp-uniform code under this predicate they get
// them directly, while code that has branched to a single lane (if (lane == 0) ...) pays a transfer per operand.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// The same with the A operand in tensor memory (lane = row, each 32-bit column two consecutive bf16 along K).
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
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
}
// 8 columns at a time: for work beside many live registers.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
// The registers of a tensor-memory load are valid only after this.
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

// Shared-memory matrix descriptor for an MN-major tile (the N or M index is contiguous in memory): rows of
// 64 contiguous MN elements (128 bytes), one row per k, 128-byte swizzle; 8 consecutive k rows form a
// 1024-byte group. `k_group_bytes`: distance between groups of 8 k rows; `mn_block_bytes`: distance between
// blocks of 64 MN elements.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t mn_block_bytes, uint32_t k_group_bytes) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>((mn_block_bytes >> 4) & 0x3FFFu) << 16) |
         (static_cast<uint64_t>((k_group_bytes >> 4) & 0x3FFFu) << 32) | (static_cast<uint64_t>(1) << 46) |
         (static_cast<uint64_t>(2) << 61);
}

// As umma_idesc, with the B operand MN-major (bit 16).
__host__ __device__ constexpr uint32_t umma_idesc_b_mn(int m, int n) { return umma_idesc(m, n) | (1u << 16); }

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Writes of this thread to shared memory become visible to the tensor core and TMA (the async proxy).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tcgen05_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Writes this warp's 32 rows x 64 bf16 columns (one row per lane, `w` = the lane's 8 x 16 bytes) through a
// swizzled shared staging area, so that each store instruction covers four whole 128-byte row pieces.
// `col0` is the first of the 64 columns, `n_valid` the number of valid output columns overall.
__device__ __forceinline__ void store_rows_bf16(const uint4 (&w)[8], unsigned char* stage, int lane, bf16* out, int ldy,
                                                int row0, int M, int col0, int n_valid) {
  uint4* st = reinterpret_cast<uint4*>(stage);
#pragma unroll
  for (int ch = 0; ch < 8; ++ch) st[lane * 8 + (ch ^ (lane & 7))] = w[ch];
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + (lane >> 3), ch = lane & 7;
    const uint4 v = st[r * 8 + (ch ^ (r & 7))];
    const int col = col0 + ch * 8;
    if (row0 + r < M && col < n_valid) *reinterpret_cast<uint4*>(out + static_cast<size_t>(row0 + r) * ldy + col) = v;
  }
  __syncwarp();
}

// As store_rows_bf16 for rows that lie anywhere: lane r holds two pieces of 32 bf16 (`lo`, `hi`: 4 x 16 bytes each)
// of its row and the row's base pointer `dst` (null: nothing is written); the pieces go to dst + off_lo and
// dst + off_hi (elements, multiples of 8). Each store instruction covers four rows' pieces of 64 bytes.
__device__ __forceinline__ void store_rows_pieces(const uint4 (&lo)[4], const uint4 (&hi)[4], unsigned char* stage, int lane,
                                                  bf16* dst, int off_lo, int off_hi) {
  uint4* st = reinterpret_cast<uint4*>(stage);
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    st[lane * 8 + (ch ^ (lane & 7))] = lo[ch];
    st[lane * 8 + ((ch + 4) ^ (lane & 7))] = hi[ch];
  }
  __syncwarp();
  const unsigned long long mine = reinterpret_cast<unsigned long long>(dst);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + (lane >> 3), ch = lane & 7;
    const uint4 v = st[r * 8 + (ch ^ (r & 7))];
    bf16* base = reinterpret_cast<bf16*>(__shfl_sync(0xffffffffu, mine, r));
    if (base != nullptr) *reinterpret_cast<uint4*>(base + (ch < 4 ? off_lo + ch * 8 : off_hi + (ch - 4) * 8)) = v;
  }
  __syncwarp();
}

// After a wait has timed out (abort_flag set by mbar_wait): before the block ends and its shared memory goes to
// another block, its copies still in flight get time to land. Bounded: about 4 ms.
__device__ __forceinline__ void drain_after_abort(volatile int* abort_flag) {
  if (*abort_flag != 0)
    for (int spin = 0; spin < (1 << 16); ++spin) __nanosleep(64);
}

// The rank of this block in its thread-block cluster, and a barrier over all threads of the cluster.
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda); nullptr if absent.
inline EncodeTiledFn tensor_map_encoder() {
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

}  // namespace dl
