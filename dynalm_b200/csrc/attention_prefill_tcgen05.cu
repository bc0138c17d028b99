// Paged flash attention for prompt portions on the 5th-generation tensor cores (tcgen05, sm_100a).
//
// One thread block per (query tile, head). A query tile is up to 128 consecutive rows of ONE request, as the
// host cuts them. Keys and values are read in place from the paged cache by TMA, 16 keys (one page, or a
// piece of a larger page) per copy, in tiles of BN keys whose boundaries are multiples of BN in absolute
// position, so the arithmetic of a row does not depend on where its portion was cut.
//
//   S = Q K^T      tcgen05.mma, M 128, N BN = 64, both operands K-major from shared memory, S in tensor memory
//   softmax        128 threads, one row each: S from tensor memory, mask by position, running maximum and
//                  sum in fp32 with base-2 exponentials, P rounded to bf16 back into tensor memory, over the
//                  first half of S's columns
//   O += P V       tcgen05.mma, M 128, N head_dim, P from tensor memory, V read as it lies in the cache
//                  (head dimension contiguous: an MN-major operand), O in tensor memory
//
// Roles: warps 0..3 softmax and the final store, warp 4 TMA producer, warp 5 issues the MMAs and owns the
// tensor-memory allocation (both run their loops as whole warps; one elected lane issues). O is rescaled only when
// a row's maximum has grown by more than 2^8 since the reference point of its exponentials was set; the result is
// the same function of the scores, with probabilities kept below 2^8.
//
// S has two buffers in tensor memory, and P takes the place of the S it was made from. The MMA warp keeps S two
// tiles ahead: behind P V of tile i it issues S of tile i + 2 into the columns that held P of tile i (the tensor
// core runs one thread's MMAs in the order of issue, so P V has read them by then). The softmax threads thus never
// wait for the tensor core in the steady state: a block's time per tile is the softmax's own (a tensor-memory
// load, 64 maxima, 64 exponentials at a quarter of a warp's issue rate, a store), and two blocks share an SM
// (its exponential unit is then busy about two thirds of the time). Tiles are 64 keys, so that S, S and O (64 + 64 + head_dim columns) leave room for two
// blocks in an SM's tensor memory at both head sizes; shared memory holds Q and three stages of K and V (two at
// head size 128, so that two blocks fit there as well).
//
// The keys of a query tile may be dealt over several blocks (`unit_parts`): with few tiles (a 512-row portion is four
// of them per head) every block would walk all of a long context's keys alone and most SMs would idle; 512 rows at
// 32,768 keys ran at 0.39 PFLOP/s against 0.63 for 2,048 rows. A tile then appears once per part in `tiles`, each
// part takes a contiguous share of the key tiles and leaves its unnormalised O, its reference point and its sum in
// scratch; the part that finds the others done (a counter per tile and head) adds them up in the order of the parts
// and stores the rows.
//
// Every wait on an mbarrier is bounded (tcgen05.cuh); on a timeout all roles fall through to the common
// exit, where tensor memory is freed, and *status tells the host.
//
// Formula and masking as the reference's attention (dynacore/cpu/cpu_device.cpp:1309-1412, 1717-1776);
// its GPU path calls ggml_flash_attn_ext here (dynacore/src/gpu/ggml_graph.cpp:465-484).
#include <limits.h>

#include "tcgen05.cuh"

namespace dl {

constexpr int FA_BM = 128;             // query rows per block
constexpr int FA_THREADS = 192;
constexpr int FA_BOX_KEYS = 16;        // keys per TMA copy
constexpr uint32_t FA_O_COL = 128;     // first tensor-memory column of O (S of even tiles from 0, of odd tiles from 64; P takes the place of S's first half)
constexpr uint32_t FA_TMEM_COLS = 256;
enum { FA_ERR_PRODUCER = 11, FA_ERR_MMA = 12, FA_ERR_SOFTMAX = 13, FA_ERR_ALIGN = 14 };

template <int HD> struct FA {
  static constexpr int BN = 64;                        // keys per tile
  static constexpr int BLOCKS_PER_SM = 2;
  static constexpr int DB = HD / 64;                   // 64-wide blocks of the head dimension (128 bytes: one swizzle row)
  static constexpr uint32_t Q_BYTES = FA_BM * HD * 2;
  static constexpr uint32_t KV_BYTES = BN * HD * 2;    // one K or one V tile
  static constexpr int STAGES = HD == 64 ? 3 : 2;      // of K and of V: 64 KiB or 96 KiB of shared memory, two blocks to an SM
  static constexpr uint32_t BAR_BYTES = 192;
  static constexpr uint32_t SMEM = Q_BYTES + 2 * STAGES * KV_BYTES + BAR_BYTES;
};

// 2^x on the special-function unit; 2^-inf = 0.
__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float fa_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// tiles[i] = (request, first row of the step, rows <= 128, first position)
template <int HD>
__global__ void __launch_bounds__(FA_THREADS, FA<HD>::BLOCKS_PER_SM)
prefill_attention_tc05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                              const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table, int max_blocks,
                              const int4* __restrict__ tiles, bf16* __restrict__ out, int out_stride, int n_heads,
                              int n_kv_heads, int page_shift, float scale_log2, int window, int* __restrict__ status,
                              const int* __restrict__ unit_parts, float* __restrict__ partial, int* __restrict__ counters,
                              int part_records) {
  constexpr int BN = FA<HD>::BN, DB = FA<HD>::DB;
  constexpr int ST = FA<HD>::STAGES;
  constexpr uint32_t Q_BYTES = FA<HD>::Q_BYTES, KV_BYTES = FA<HD>::KV_BYTES;
  constexpr uint32_t Q_BLOCK = FA_BM * 128;       // bytes of one 64-wide block of Q (128 rows of 128 bytes)
  constexpr uint32_t KV_BLOCK = BN * 128;         // likewise for a K or V tile
  extern __shared__ __align__(1024) unsigned char fa_raw[];
  unsigned char* q_s = fa_raw;
  unsigned char* k_s = q_s + Q_BYTES;             // [ST][KV_BYTES]; the output staging at the end
  unsigned char* v_s = k_s + ST * KV_BYTES;       // [ST][KV_BYTES]
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + ST * KV_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                    // [ST]
  uint64_t* v_full = k_full + ST;                 // [ST]
  uint64_t* k_empty = v_full + ST;                // [ST] S of the tile has been computed
  uint64_t* v_empty = k_empty + ST;               // [ST] P V of the tile has been computed
  uint64_t* s_full = v_empty + ST;                // [2] S of a tile is in its buffer
  uint64_t* p_full = s_full + 2;                  // [2] P has taken its place and O has been rescaled
  uint64_t* pv_done = s_full + 4;                 // O includes the tile (one phase per tile)
  uint64_t* o_done = s_full + 5;                  // O includes the last tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (smem_u32(fa_raw) & 1023u) {                 // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicExch(status, FA_ERR_ALIGN);
    return;
  }

  const int4 tile = ck_tile(tiles[blockIdx.y]);      // heads of one tile are neighbours in launch order: the tiles with most keys start first
  const int req = tile.x, row0 = tile.y, nrows = tile.z, pos0 = tile.w;
  if (nrows <= 0) return;                   // (a tile that a checked build has refused; nothing is set up yet)
  const int head = blockIdx.x;
  const int kvh = head / (n_heads / n_kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos_last = pos0 + nrows - 1;
  const int lo_tile = window > 0 ? max(0, pos0 - window + 1) : 0;      // the first key any row of the tile reads
  int j_begin = lo_tile / BN, n_kt = pos_last / BN - j_begin + 1;
  // this block's share of the tile's keys: part `part` of `parts` (word = part | parts << 8 | first scratch slot << 16)
  const int part_word = unit_parts != nullptr ? ck_part_word(unit_parts[blockIdx.y], part_records) : 0;
  const int part = part_word & 0xff, parts = (part_word >> 8) & 0xff, slot0 = part_word >> 16;
  if (parts > 1) {
    const int per = (n_kt + parts - 1) / parts;
    j_begin += part * per;
    n_kt = max(0, min(per, n_kt - part * per));
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < ST; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], 128);
    }
    mbar_init(pv_done, 1);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(FA_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_before_sync();
  __syncthreads();
  tcgen05_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // up to here the block may have run beside the end of the kernel in front (programmatic dependent launch); q and the
  // newest keys come from that kernel
  pdl_wait();
  pdl_trigger();

  if (warp == 4) {
    // TMA producer: the whole warp runs the loop, one elected lane issues the copies
    const int* table = block_table + static_cast<size_t>(req) * max_blocks;
    const int page_mask = (1 << page_shift) - 1;
    if (elect_one()) {
      mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int db = 0; db < DB; ++db) tma_load_2d(q_s + db * Q_BLOCK, &map_q, head * HD + db * 64, row0, q_full);
    }
    // a piece of 16 keys wholly outside [lo_tile, pos_last] is masked anyway: it is read from the nearest
    // piece inside, so that every copy reads pages this request holds (finite values)
    const int first_piece = lo_tile & ~(FA_BOX_KEYS - 1), last_piece = pos_last & ~(FA_BOX_KEYS - 1);
    for (int i = 0; i < n_kt; ++i) {
      const int s = i % ST;
      const uint32_t round = static_cast<uint32_t>(i / ST);
      // lane b looks up the page of piece b
      int my_slot = 0;
      if (lane < BN / FA_BOX_KEYS) {
        const int key = min(max((j_begin + i) * BN + lane * FA_BOX_KEYS, first_piece), last_piece);
        my_slot = (ck_page(table, key >> page_shift, max_blocks) << page_shift) + (key & page_mask);
      }
      if (i >= ST && !warp_wait(&k_empty[s], (round & 1) ^ 1, status, FA_ERR_PRODUCER, abort_flag)) break;
      if (elect_one()) mbar_expect_tx(&k_full[s], KV_BYTES);
#pragma unroll
      for (int b = 0; b < BN / FA_BOX_KEYS; ++b) {
        const int slot = __shfl_sync(0xffffffffu, my_slot, b);
        if (elect_one()) {
#pragma unroll
          for (int db = 0; db < DB; ++db)
            tma_load_3d(k_s + s * KV_BYTES + db * KV_BLOCK + b * (FA_BOX_KEYS * 128), &map_k, db * 64, kvh, slot, &k_full[s]);
        }
      }
      if (i >= ST && !warp_wait(&v_empty[s], (round & 1) ^ 1, status, FA_ERR_PRODUCER, abort_flag)) break;
      if (elect_one()) mbar_expect_tx(&v_full[s], KV_BYTES);
#pragma unroll
      for (int b = 0; b < BN / FA_BOX_KEYS; ++b) {
        const int slot = __shfl_sync(0xffffffffu, my_slot, b);
        if (elect_one()) {
#pragma unroll
          for (int db = 0; db < DB; ++db)
            tma_load_3d(v_s + s * KV_BYTES + db * KV_BLOCK + b * (FA_BOX_KEYS * 128), &map_v, db * 64, kvh, slot, &v_full[s]);
        }
      }
    }
    if (*abort_flag) {
      // Another role gave up: before the block ends, give the copies in flight time to land (bounded).
      for (int spin = 0; spin < (1 << 16); ++spin) __nanosleep(64);
    }
  } else if (warp == 5) {
    // MMA issue: the whole warp runs the loop, one elected lane issues the instructions
    constexpr uint32_t idesc_s = umma_idesc(FA_BM, BN);
    constexpr uint32_t idesc_o = umma_idesc_b_mn(FA_BM, HD);
    // descriptors of the first pieces; a step along the tile adds (bytes >> 4) to the address field
    const uint64_t q_desc = umma_desc_sw128(smem_u32(q_s)), k_desc = umma_desc_sw128(smem_u32(k_s));
    const uint64_t v_desc = umma_desc_mn_sw128(smem_u32(v_s), KV_BLOCK, 1024);
    // S of tile i: waits for K, issues HD / 16 MMAs, frees the K stage and signals the softmax warps
    auto issue_s = [&](int i) -> bool {
      const int s = i % ST;
      if (!warp_wait(&k_full[s], (i / ST) & 1, status, FA_ERR_MMA, abort_flag)) return false;
      tcgen05_after_sync();
      if (elect_one()) {
#pragma unroll
        for (int db = 0; db < DB; ++db)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base + (i & 1) * BN, q_desc + ((db * Q_BLOCK + k * 32) >> 4),
                      k_desc + ((s * KV_BYTES + db * KV_BLOCK + k * 32) >> 4), idesc_s, (db > 0 || k > 0) ? 1u : 0u);
        umma_commit(&k_empty[s]);
        umma_commit(&s_full[i & 1]);
      }
      __syncwarp();
      return true;
    };
    bool ok = warp_wait(q_full, 0, status, FA_ERR_MMA, abort_flag);
    if (n_kt > 0) ok = ok && issue_s(0);
    if (n_kt > 1) ok = ok && issue_s(1);
    for (int i = 0; i < n_kt && ok; ++i) {
      const int s = i % ST;
      if (!warp_wait(&v_full[s], (i / ST) & 1, status, FA_ERR_MMA, abort_flag)) break;
      if (!warp_wait(&p_full[i & 1], (i >> 1) & 1, status, FA_ERR_MMA, abort_flag)) break;
      tcgen05_after_sync();
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          // P: 16 keys = 8 tensor-memory columns (two bf16 each). V: 16 keys = 16 rows of 128 bytes; groups of 8
          // keys 1024 bytes apart, blocks of 64 head dimensions KV_BLOCK apart.
          umma_bf16_ts(tmem_base + FA_O_COL, tmem_base + (i & 1) * BN + kk * 8,
                       v_desc + ((s * KV_BYTES + kk * (16 * 128)) >> 4), idesc_o, (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[s]);
        umma_commit(pv_done);
        if (i + 1 == n_kt) umma_commit(o_done);
      }
      __syncwarp();
      // S of the tile after the next goes where P of this one lies: issued behind the MMAs that read it
      if (i + 2 < n_kt && !issue_s(i + 2)) break;
    }
  } else {
    // softmax: thread r owns query row r = tensor-memory lane r
    const int r = threadIdx.x;
    const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const uint32_t taddr_o = taddr_row + FA_O_COL;
    const int pos_r = pos0 + r;
    const int lo_r = window > 0 ? max(0, pos_r - window + 1) : 0;
    float m_ref = -INFINITY;      // the reference point of this row's exponentials, in base-2 units
    float l_run = 0.0f;
    bool ok = true;
    for (int i = 0; i < n_kt; ++i) {
      const uint32_t taddr_s = taddr_row + (i & 1) * BN;
      if (!warp_wait(&s_full[i & 1], (i >> 1) & 1, status, FA_ERR_SOFTMAX, abort_flag)) { ok = false; break; }
      tcgen05_after_sync();
      uint32_t sv[BN];
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 32) tmem_ld32(taddr_s + c0, *reinterpret_cast<uint32_t(*)[32]>(&sv[c0]));
      tmem_ld_wait();

      const int key0 = (j_begin + i) * BN;
      const bool edge = key0 + BN - 1 > pos0 + warp * 32 || (window > 0 && key0 < max(0, pos0 + warp * 32 + 31 - window + 1));
      if (edge) {
#pragma unroll
        for (int c = 0; c < BN; ++c) {
          const int key = key0 + c;
          if (key > pos_r || key < lo_r) sv[c] = 0xff800000u;      // -inf
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int c = 0; c < BN; c += 8) {
        mx0 = fa_max3(mx0, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]));
        mx1 = fa_max3(mx1, __uint_as_float(sv[c + 2]), __uint_as_float(sv[c + 3]));
        mx2 = fa_max3(mx2, __uint_as_float(sv[c + 4]), __uint_as_float(sv[c + 5]));
        mx3 = fa_max3(mx3, __uint_as_float(sv[c + 6]), __uint_as_float(sv[c + 7]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2;      // the scale is positive
      float corr = 1.0f;
      bool rescale = false;
      if (m_ref == -INFINITY) {
        m_ref = mx;                 // nothing accumulated so far (may stay -inf: no visible key yet)
      } else if (mx > m_ref + 8.0f) {
        corr = fa_exp2(m_ref - mx);
        m_ref = mx;
        rescale = true;
      }
      if (__any_sync(0xffffffffu, rescale)) {
        // O must hold every tile before this one. S of this tile was committed behind P V of tile i - 2, so that one
        // is complete and the barrier is in the phase of tile i - 1 or past it: its parity cannot be mistaken.
        if (!warp_wait(pv_done, (i - 1) & 1, status, FA_ERR_SOFTMAX, abort_flag)) { ok = false; break; }
        tcgen05_after_sync();
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 8) {          // a few columns at a time: S stays in its registers
          uint32_t o[8];
          tmem_ld8(taddr_o + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 8; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * corr);
          tmem_st8(taddr_o + c0, o);
        }
      }
      const float neg_m = m_ref == -INFINITY ? 0.0f : -m_ref;
      float sum0 = 0.0f, sum1 = 0.0f;
      // P in tensor memory: this thread's lane, column j = keys 2j and 2j + 1, over the first half of S
      uint32_t pk[BN / 2];
#pragma unroll
      for (int c = 0; c < BN; c += 2) {
        const float p0 = fa_exp2(fmaf(__uint_as_float(sv[c]), scale_log2, neg_m));
        const float p1 = fa_exp2(fmaf(__uint_as_float(sv[c + 1]), scale_log2, neg_m));
        sum0 += p0;
        sum1 += p1;
        pk[c / 2] = pack2_bf16(p0, p1);
      }
      tmem_st32(taddr_s, pk);
      tmem_st_wait();
      l_run = l_run * corr + (sum0 + sum1);
      tcgen05_before_sync();
      mbar_arrive(&p_full[i & 1]);
    }
    // (a part without key tiles has nothing to wait for: its O counts as zero)
    ok = ok && (n_kt == 0 || warp_wait(o_done, 0, status, FA_ERR_SOFTMAX, abort_flag));
    if (ok) tcgen05_after_sync();
    unsigned char* my_stage = k_s + warp * 4096;      // every K and V stage has been consumed
    if (parts <= 1) {
      if (ok) {
        const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 64) {
          uint4 w[8];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t v[32];
            tmem_ld32(taddr_o + c0 + hh * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; j += 8)
              w[hh * 4 + j / 8] = make_uint4(pack2_bf16(__uint_as_float(v[j]) * inv, __uint_as_float(v[j + 1]) * inv),
                                             pack2_bf16(__uint_as_float(v[j + 2]) * inv, __uint_as_float(v[j + 3]) * inv),
                                             pack2_bf16(__uint_as_float(v[j + 4]) * inv, __uint_as_float(v[j + 5]) * inv),
                                             pack2_bf16(__uint_as_float(v[j + 6]) * inv, __uint_as_float(v[j + 7]) * inv));
          }
          store_rows_bf16(w, my_stage, lane, out, out_stride, row0 + warp * 32, row0 + nrows, head * HD + c0, INT_MAX);
        }
      }
    } else {
      // This part's record: [head_dim + 2][128 rows] floats (a column of 128 rows is contiguous: the threads of a warp
      // write and read neighbouring words): unnormalised O, then the reference point and the sum of each row.
      constexpr int REC = (HD + 2) * FA_BM;
      float* mine = partial + (static_cast<size_t>(slot0 + part) * n_heads + head) * REC;
      if (ok) {
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t v[32];
          if (n_kt > 0) {
            tmem_ld32(taddr_o + c0, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) mine[(c0 + j) * FA_BM + r] = __uint_as_float(v[j]);
        }
        mine[HD * FA_BM + r] = m_ref;
        mine[(HD + 1) * FA_BM + r] = l_run;
        __threadfence();
      }
      // The four softmax warps meet (every one of them gets here, whatever happened before); the part that finds all
      // others done adds the parts up, in the order of the parts whoever came last, and stores the rows.
      __shared__ int s_last;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 0) {
        int last = 0;
        if (*abort_flag == 0) {
          int* counter = counters + slot0 * n_heads + head;
          last = atomicAdd(counter, 1) == parts - 1;
          if (last) *counter = 0;               // ready for the next launch
        }
        s_last = last;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (s_last) {
        __threadfence();
        const float* first = partial + (static_cast<size_t>(slot0) * n_heads + head) * REC;
        const size_t step = static_cast<size_t>(n_heads) * REC;          // from one part's record to the next
        float m = -INFINITY;
        for (int p = 0; p < parts; ++p) m = fmaxf(m, __ldcg(first + p * step + HD * FA_BM + r));
        float l = 0.0f;
        for (int p = 0; p < parts; ++p) {
          const float mp = __ldcg(first + p * step + HD * FA_BM + r);
          l += mp == -INFINITY ? 0.0f : __ldcg(first + p * step + (HD + 1) * FA_BM + r) * fa_exp2(mp - m);
        }
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 64) {
          uint4 w[8];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            float acc[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = 0.0f;
            for (int p = 0; p < parts; ++p) {
              const float mp = __ldcg(first + p * step + HD * FA_BM + r);
              const float sc = mp == -INFINITY ? 0.0f : fa_exp2(mp - m);
              const float* src = first + p * step + static_cast<size_t>(c0 + hh * 32) * FA_BM + r;
#pragma unroll
              for (int j = 0; j < 32; ++j) acc[j] = fmaf(sc, __ldcg(src + j * FA_BM), acc[j]);
            }
#pragma unroll
            for (int j = 0; j < 32; j += 8)
              w[hh * 4 + j / 8] = make_uint4(pack2_bf16(acc[j] * inv, acc[j + 1] * inv), pack2_bf16(acc[j + 2] * inv, acc[j + 3] * inv),
                                             pack2_bf16(acc[j + 4] * inv, acc[j + 5] * inv), pack2_bf16(acc[j + 6] * inv, acc[j + 7] * inv));
          }
          store_rows_bf16(w, my_stage, lane, out, out_stride, row0 + warp * 32, row0 + nrows, head * HD + c0, INT_MAX);
        }
      }
    }
  }
  // common exit: every role arrives here, with or without a timeout
  tcgen05_before_sync();
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(FA_TMEM_COLS) : "memory");
  }
}

// ---- host side -------------------------------------------------------------------------------------

// q: [n_rows, cols] bf16 with a row pitch of `ld` elements; box = 128 rows x 64 columns.
static int make_q_map(CUtensorMap* map, const void* base, int n_rows, int cols, int ld) {
  EncodeTiledFn fn = tensor_map_encoder();
  if (fn == nullptr) return DL_ERR_UNSUPPORTED;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(n_rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {64, FA_BM};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 700000 + static_cast<int>(r);
}

// cache: [n_slots, n_kv_heads, head_dim] bf16, contiguous; box = 16 slots x 1 head x 64 columns.
static int make_cache_map(CUtensorMap* map, const void* base, long long n_slots, int n_kv_heads, int head_dim) {
  EncodeTiledFn fn = tensor_map_encoder();
  if (fn == nullptr) return DL_ERR_UNSUPPORTED;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(n_kv_heads), static_cast<cuuint64_t>(n_slots)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_dim) * 2, static_cast<cuuint64_t>(n_kv_heads) * head_dim * 2};
  const cuuint32_t box[3] = {64, 1, FA_BOX_KEYS};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 700000 + static_cast<int>(r);
}

template <int HD>
int launch_prefill_tc05(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const int* block_table,
                        int max_blocks, const int* tiles, int n_tiles, void* out, int out_stride, int n_heads, int n_kv_heads,
                        int page_shift, float scale, int window, int* status, const int* unit_parts, float* partial, int* counters,
                        int part_records, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc05_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(FA<HD>::SMEM));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  dim3 grid(n_heads, n_tiles);
  return launch_streaming(prefill_attention_tc05_kernel<HD>, grid, dim3(FA_THREADS), FA<HD>::SMEM, stream, mq, mk, mv, block_table,
                          max_blocks, reinterpret_cast<const int4*>(tiles), static_cast<bf16*>(out), out_stride, n_heads,
                          n_kv_heads, page_shift, scale * 1.4426950408889634f, window, status, unit_parts, partial, counters, part_records);
}

}  // namespace dl

// bfloat16, head_dim 64 or 128, pages of 16 keys or a larger power of two. q: [n_rows, q_stride] with head h at
// column h * head_dim; caches: [n_pages, page_size, n_kv_heads, head_dim] contiguous and free of NaN/Inf bit
// patterns (a fresh cache is zero-filled); tiles: int32 [n_tiles, 4] = (request, first row, rows <= 128, first
// position), 16-byte aligned. status: one device int, set to a nonzero code if a wait inside the kernel timed
// out (left untouched otherwise). Other shapes return "unsupported": the caller has the mma.sync kernel.
// unit_parts (or null: every tile is whole): int32 [n_tiles], for a tile whose keys are dealt over several entries of
// `tiles` (equal in their four numbers) which part this entry is: part | parts << 8 | slot << 16, parts up to 255, 0 or
// 1 = whole; the parts of a tile use the records slot .. slot + parts - 1 of `partial` (float32, (slots in use) *
// n_heads * (head_dim + 2) * 128 elements) and the counters slot * n_heads .. + n_heads - 1 of `counters` (int32, zero
// before the first launch; the kernel leaves them zero unless a wait timed out). part_records: how many records
// `partial` holds (what a checked build compares the words with).
DL_EXPORT int dl_paged_attention_prefill_tcgen05(const void* q, int q_stride, int n_rows, const void* k_cache,
                                                 const void* v_cache, long long n_pages, const int* block_table,
                                                 int max_blocks, const int* tiles, int n_tiles, void* out, int out_stride,
                                                 int n_heads, int n_kv_heads, int head_dim, int page_size, float scale,
                                                 int window, int* status, const int* unit_parts, float* partial,
                                                 int* counters, int part_records, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  if ((1 << page_shift) != page_size || page_size < dl::FA_BOX_KEYS || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 ||
      n_tiles > 65535 || (head_dim != 64 && head_dim != 128) || (q_stride & 7) || (out_stride & 7) || !(scale > 0.0f) ||
      (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
      (reinterpret_cast<uintptr_t>(k_cache) & 15) || (reinterpret_cast<uintptr_t>(v_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(tiles) & 15) || status == nullptr || n_rows <= 0 || n_pages <= 0 ||
      n_pages * page_size > 0x7fffffffll || (unit_parts != nullptr && (partial == nullptr || counters == nullptr)))
    return DL_ERR_UNSUPPORTED;
  CUtensorMap mq, mk, mv;
  int rc = dl::make_q_map(&mq, q, n_rows, n_heads * head_dim, q_stride);
  if (rc != 0) return rc;
  rc = dl::make_cache_map(&mk, k_cache, n_pages * page_size, n_kv_heads, head_dim);
  if (rc != 0) return rc;
  rc = dl::make_cache_map(&mv, v_cache, n_pages * page_size, n_kv_heads, head_dim);
  if (rc != 0) return rc;
  if (head_dim == 64)
    return dl::launch_prefill_tc05<64>(mq, mk, mv, block_table, max_blocks, tiles, n_tiles, out, out_stride, n_heads,
                                       n_kv_heads, page_shift, scale, window, status, unit_parts, partial, counters, part_records, stream);
  return dl::launch_prefill_tc05<128>(mq, mk, mv, block_table, max_blocks, tiles, n_tiles, out, out_stride, n_heads,
                                      n_kv_heads, page_shift, scale, window, status, unit_parts, partial, counters, part_records, stream);
}
