// Split-KV paged attention for rows that bring few tokens (decode): bandwidth-bound, CUDA cores.
//
// One thread block per (key split, KV head, row). The block streams its share of the row's keys and
// values once and serves every query head of the KV head's group from them (the reference's
// GQA-grouped pass, dynacore/cpu/cpu_device.cpp:1297-1308,1347-1352). Inside a warp, LPK lanes share
// one key: each lane holds one 16-byte vector of the head dimension, so a warp instruction reads
// 32 / LPK whole key rows, fully coalesced. Scores are reduced over those lanes by shuffles; the
// running (max, sum, acc) of the online softmax is kept per lane in fp32 and merged at the end over
// the warp's key slots, then over the block's warps in shared memory. With more than one split the
// block writes its unnormalised (acc, max, sum) to scratch and `attention_combine_kernel` merges the
// splits by the log-sum-exp rule of the reference's split-K variant (:1782-1845); the tensor-core variant
// instead launches the splits of a row as one thread-block cluster and merges them in the shared memory of
// the cluster's first block.
//
// Scratch layout: part[((row * n_heads + head) * n_split + split) * (head_dim + 2)] = acc[head_dim], max, sum.
#include <cooperative_groups.h>

#include "common.cuh"

namespace dl {

constexpr int DEC_THREADS = 128;
constexpr int DEC_WARPS = DEC_THREADS / 32;
constexpr int DEC_G = 4;   // query heads of one group served per block
constexpr int DEC_U = 4;   // keys in flight per lane group

template <typename T, int LPK>
__global__ void __launch_bounds__(DEC_THREADS)
decode_attention_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                        const T* __restrict__ v_cache, const int* __restrict__ block_table, int max_blocks,
                        const int* __restrict__ positions, const int* __restrict__ row_request,
                        T* __restrict__ out, int out_stride, float* __restrict__ part, int n_heads, int n_kv_heads,
                        int head_dim, int page_shift, float scale_log2, int window, int n_split) {
  constexpr int V = PerVec<T>::n;
  constexpr int KPW = 32 / LPK;
  extern __shared__ float sm[];   // [DEC_WARPS][DEC_G][head_dim + 2]
  const int split = blockIdx.x, row = blockIdx.z;
  const int group = n_heads / n_kv_heads;
  const int chunks = (group + DEC_G - 1) / DEC_G;
  const int kvh = blockIdx.y / chunks, h0 = (blockIdx.y % chunks) * DEC_G;
  const int ng = min(DEC_G, group - h0);
  const int head0 = kvh * group + h0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kg = lane / LPK, dl_ = lane % LPK;
  const bool dim_ok = dl_ * V < head_dim;
  const int page_mask = (1 << page_shift) - 1;

  const int pos = positions[row];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int n = pos + 1 - lo;
  int len = (n + n_split - 1) / n_split;
  len = (len + 15) & ~15;
  const int k_begin = lo + split * len;
  const int k_end = min(pos + 1, k_begin + len);
  const int* table = block_table + static_cast<size_t>(ck_request(row_request[row])) * max_blocks;
  const size_t kv_row = static_cast<size_t>(n_kv_heads) * head_dim;
  const size_t head_off = static_cast<size_t>(kvh) * head_dim + dl_ * V;

  float qv[DEC_G][V];
  float acc[DEC_G][V];
  float m[DEC_G], l[DEC_G];
#pragma unroll
  for (int g = 0; g < DEC_G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.0f;
#pragma unroll
    for (int j = 0; j < V; ++j) { acc[g][j] = 0.0f; qv[g][j] = 0.0f; }
    if (g < ng && dim_ok) {
      const T* qp = q + static_cast<size_t>(row) * q_stride + static_cast<size_t>(head0 + g) * head_dim + dl_ * V;
      float f[V];
      unpack<T>(*reinterpret_cast<const Vec16*>(qp), f);
#pragma unroll
      for (int j = 0; j < V; ++j) qv[g][j] = f[j] * scale_log2;
    }
  }

  constexpr int STRIDE = DEC_WARPS * KPW;   // keys between a lane group's consecutive keys
  // The loop bound is the same for every lane of a warp (the shuffles below name all 32 lanes);
  // a lane group whose key lies past the end computes on zeros and discards the score.
  for (int base = k_begin + warp * KPW; base < k_end; base += STRIDE * DEC_U) {
    const int t0 = base + kg;
    Vec16 kr[DEC_U], vr[DEC_U];
    bool ok[DEC_U];
#pragma unroll
    for (int u = 0; u < DEC_U; ++u) {
      const int t = t0 + u * STRIDE;
      ok[u] = t < k_end;
      kr[u].raw = make_uint4(0, 0, 0, 0);
      vr[u].raw = make_uint4(0, 0, 0, 0);
      if (ok[u] && dim_ok) {
        const size_t slot = (static_cast<size_t>(ck_page(table, t >> page_shift, max_blocks)) << page_shift) + (t & page_mask);
        kr[u] = *reinterpret_cast<const Vec16*>(k_cache + slot * kv_row + head_off);
        vr[u] = *reinterpret_cast<const Vec16*>(v_cache + slot * kv_row + head_off);
      }
    }
    float s[DEC_G][DEC_U];
#pragma unroll
    for (int u = 0; u < DEC_U; ++u) {
      float kf[V];
      unpack<T>(kr[u], kf);
#pragma unroll
      for (int g = 0; g < DEC_G; ++g) {
        float d = 0.0f;
        if (g < ng) {
#pragma unroll
          for (int j = 0; j < V; ++j) d = fmaf(qv[g][j], kf[j], d);
        }
        s[g][u] = d;
      }
    }
#pragma unroll
    for (int o = 1; o < LPK; o <<= 1) {
#pragma unroll
      for (int g = 0; g < DEC_G; ++g) {
        if (g < ng) {
#pragma unroll
          for (int u = 0; u < DEC_U; ++u) s[g][u] += __shfl_xor_sync(0xffffffffu, s[g][u], o);
        }
      }
    }
    float vf[DEC_U][V];
#pragma unroll
    for (int u = 0; u < DEC_U; ++u) unpack<T>(vr[u], vf[u]);
#pragma unroll
    for (int g = 0; g < DEC_G; ++g) {
      if (g < ng) {
        float bm = -INFINITY;
#pragma unroll
        for (int u = 0; u < DEC_U; ++u) {
          if (!ok[u]) s[g][u] = -INFINITY;
          bm = fmaxf(bm, s[g][u]);
        }
        if (bm > -INFINITY) {                      // this lane group had at least one key in range
          const float m_new = fmaxf(m[g], bm);
          const float corr = exp2f(m[g] - m_new);  // 0 the first time
          float p[DEC_U], ps = 0.0f;
#pragma unroll
          for (int u = 0; u < DEC_U; ++u) {
            p[u] = exp2f(s[g][u] - m_new);
            ps += p[u];
          }
          l[g] = l[g] * corr + ps;
          m[g] = m_new;
#pragma unroll
          for (int j = 0; j < V; ++j) {
            float a = acc[g][j] * corr;
#pragma unroll
            for (int u = 0; u < DEC_U; ++u) a = fmaf(p[u], vf[u][j], a);
            acc[g][j] = a;
          }
        }
      }
    }
  }

  // merge the warp's key slots (lanes that differ in kg)
#pragma unroll
  for (int o = LPK; o < 32; o <<= 1) {
#pragma unroll
    for (int g = 0; g < DEC_G; ++g) {
      if (g < ng) {
        const float om = __shfl_xor_sync(0xffffffffu, m[g], o);
        const float ol = __shfl_xor_sync(0xffffffffu, l[g], o);
        const float m_new = fmaxf(m[g], om);
        const float ca = m_new == -INFINITY ? 0.0f : exp2f(m[g] - m_new);
        const float cb = m_new == -INFINITY ? 0.0f : exp2f(om - m_new);
        l[g] = l[g] * ca + ol * cb;
        m[g] = m_new;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float oa = __shfl_xor_sync(0xffffffffu, acc[g][j], o);
          acc[g][j] = acc[g][j] * ca + oa * cb;
        }
      }
    }
  }
  const int rec = head_dim + 2;
  if (kg == 0) {
#pragma unroll
    for (int g = 0; g < DEC_G; ++g) {
      if (g < ng) {
        float* dst = sm + (static_cast<size_t>(warp) * DEC_G + g) * rec;
        if (dim_ok) {
#pragma unroll
          for (int j = 0; j < V; ++j) dst[dl_ * V + j] = acc[g][j];
        }
        if (dl_ == 0) {
          dst[head_dim] = m[g];
          dst[head_dim + 1] = l[g];
        }
      }
    }
  }
  __syncthreads();
  // merge the block's warps: one thread per (head, dim)
  for (int idx = threadIdx.x; idx < ng * head_dim; idx += DEC_THREADS) {
    const int g = idx / head_dim, d = idx % head_dim;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, sm[(w * DEC_G + g) * rec + head_dim]);
    float a = 0.0f, ll = 0.0f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float* src = sm + (w * DEC_G + g) * rec;
      const float c = mm == -INFINITY ? 0.0f : exp2f(src[head_dim] - mm);
      a += src[d] * c;
      ll += src[head_dim + 1] * c;
    }
    const int head = head0 + g;
    if (n_split == 1) {
      out[static_cast<size_t>(row) * out_stride + static_cast<size_t>(head) * head_dim + d] = from_float<T>(a / ll);
    } else {
      float* dst = part + ((static_cast<size_t>(row) * n_heads + head) * n_split + split) * rec;
      dst[d] = a;
      if (d == 0) {
        dst[head_dim] = mm;
        dst[head_dim + 1] = ll;
      }
    }
  }
}

template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ part, T* __restrict__ out, int out_stride,
                                         int n_heads, int head_dim, int n_split) {
  pdl_wait();
  pdl_trigger();
  const int head = blockIdx.x, row = blockIdx.y;
  const int rec = head_dim + 2;
  const float* base = part + (static_cast<size_t>(row) * n_heads + head) * n_split * rec;
  float mm = -INFINITY;
  for (int s = 0; s < n_split; ++s) mm = fmaxf(mm, base[s * rec + head_dim]);
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float a = 0.0f, ll = 0.0f;
    for (int s = 0; s < n_split; ++s) {
      const float ms = base[s * rec + head_dim];
      const float c = ms == -INFINITY ? 0.0f : exp2f(ms - mm);
      a += base[s * rec + d] * c;
      ll += base[s * rec + head_dim + 1] * c;
    }
    out[static_cast<size_t>(row) * out_stride + static_cast<size_t>(head) * head_dim + d] = from_float<T>(a / ll);
  }
}

template <typename T>
int launch_decode(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table,
                  int max_blocks, const int* positions, const int* row_request, void* out, int out_stride,
                  float* part, int rows, int n_heads, int n_kv_heads, int head_dim, int page_size, float scale,
                  int window, int n_split, cudaStream_t stream) {
  constexpr int V = PerVec<T>::n;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  if ((1 << page_shift) != page_size) return DL_ERR_UNSUPPORTED;
  if (head_dim % 16 != 0 || head_dim <= 0 || head_dim > 32 * V || n_heads % n_kv_heads != 0 || n_split < 1 ||
      rows > 65535 || (n_split > 1 && part == nullptr))
    return DL_ERR_UNSUPPORTED;
  const int vecs = head_dim / V + (head_dim % V ? 1 : 0);
  int lpk = 1;
  while (lpk < vecs) lpk <<= 1;
  const int group = n_heads / n_kv_heads;
  const int chunks = (group + DEC_G - 1) / DEC_G;
  dim3 grid(n_split, n_kv_heads * chunks, rows);
  const size_t smem = static_cast<size_t>(DEC_WARPS) * DEC_G * (head_dim + 2) * sizeof(float);
  const float scale_log2 = scale * 1.4426950408889634f;
#define DL_LAUNCH(L)                                                                                            \
  decode_attention_kernel<T, L><<<grid, DEC_THREADS, smem, stream>>>(                                           \
      static_cast<const T*>(q), q_stride, static_cast<const T*>(kc), static_cast<const T*>(vc), block_table,    \
      max_blocks, positions, row_request, static_cast<T*>(out), out_stride, part, n_heads, n_kv_heads, head_dim, \
      page_shift, scale_log2, window, n_split)
  switch (lpk) {
    case 1: DL_LAUNCH(1); break;
    case 2: DL_LAUNCH(2); break;
    case 4: DL_LAUNCH(4); break;
    case 8: DL_LAUNCH(8); break;
    case 16: DL_LAUNCH(16); break;
    case 32: DL_LAUNCH(32); break;
    default: return DL_ERR_UNSUPPORTED;
  }
#undef DL_LAUNCH
  int rc = launch_status();
  if (rc != 0 || n_split == 1) return rc;
  dim3 cgrid(n_heads, rows);
  const int cthreads = head_dim <= 32 ? 32 : (head_dim <= 64 ? 64 : 128);
  attention_combine_kernel<T><<<cgrid, cthreads, 0, stream>>>(part, static_cast<T*>(out), out_stride, n_heads,
                                                             head_dim, n_split);
  return launch_status();
}


// ------------------------------------------------------------------------------------------------
// The tensor-core variant (bf16): the same split-KV scheme, but the group's query heads form the
// rows of an m16n8k16 tile, and each warp streams its own key tiles through a private multi-stage
// cp.async pipeline in shared memory, so that many kilobytes stay in flight per warp whatever the
// register budget. Warp w of a block's W warps takes key tiles w, w + W, ... of the block's key range; tiles are
// KT keys. Scores, softmax and the merge are fp32; P is rounded to bf16 for the P V product.
// A warp's tiles are a chain of dependent work (copy, Q K^T, softmax, P V), so a block's time is the length of
// that chain: eight warps with tiles of 16 keys halve it against four warps with tiles of 32 at the same shared
// memory. Groups of up to 8 query heads (every Llama shape) use rows 0 to 7 of the 16-row tile only, and the
// softmax and rescaling of rows 8 to 15 are left out.
// ------------------------------------------------------------------------------------------------

__device__ __forceinline__ void dt_cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void dt_ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void dt_ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void dt_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float dt_exp2(float x) {     // one special-function instruction; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t dt_pack(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

template <int HD, int STAGES, int KT, int W>
__global__ void __launch_bounds__(W * 32)
decode_attention_tc_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ k_cache,
                           const bf16* __restrict__ v_cache, const int* __restrict__ block_table, int max_blocks,
                           const int* __restrict__ positions, const int* __restrict__ row_request,
                           bf16* __restrict__ out, int out_stride, float* __restrict__ part, int n_heads,
                           int n_kv_heads, int page_shift, float scale_log2, int window, int n_split,
                           int cluster_merge, int xbuf_offset, const void* __restrict__ ahead, long long ahead_bytes,
                           const int* __restrict__ plan, int* __restrict__ counters, int part_stride) {
  l2_prefetch_share(ahead, ahead_bytes);     // what the kernel after this one will stream (see common.cuh)
  constexpr int LD = HD + 8;
  constexpr int CH = HD / 8;
  constexpr int KS = HD / 16;
  constexpr int TILE_ELEMS = KT * LD;                 // one of K or V of one stage
  constexpr int DT_WARPS = W, DT_THREADS = W * 32;
  extern __shared__ __align__(16) unsigned char dt_smem[];
  bf16* Qs = reinterpret_cast<bf16*>(dt_smem);           // [16][LD]
  bf16* KV = Qs + 16 * LD;                               // [warp][stage][K | V][KT][LD]
  float* merge = reinterpret_cast<float*>(dt_smem);      // reused after the loop: [warp][16][HD + 2]

  // Which keys of which row this block takes. Without a plan the grid says it: (split, KV head and chunk of its
  // group, row), every row cut into n_split parts. With a plan (see dl_paged_attention_decode_planned) the host has
  // dealt the keys of all rows into units of about equal size, one block each: int4 (row, KV head chunk, part, parts of
  // that row), after a header whose first word is the number of units; blocks past it have nothing to do.
  int split = blockIdx.x, row = blockIdx.z, ychunk = blockIdx.y;
  if (plan != nullptr) {
    if (static_cast<int>(blockIdx.x) >= plan[0]) return;
    const int4 unit = reinterpret_cast<const int4*>(plan)[1 + blockIdx.x];
    row = ck_row(unit.x);
    ychunk = unit.y;
    split = unit.z;
    n_split = unit.w;
  }
  const int group = n_heads / n_kv_heads;
  const int chunks = (group + 15) / 16;
  const int kvh = ychunk / chunks, h0 = (ychunk % chunks) * 16;
  const int ng = min(16, group - h0);
  const bool wide = ng > 8;                           // rows 8 to 15 of the tile hold query heads too
  const int head0 = kvh * group + h0;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int page_mask = (1 << page_shift) - 1;

  const int pos = positions[row];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int n = pos + 1 - lo;
  int len = (n + n_split - 1) / n_split;
  len = (len + KT - 1) / KT * KT;
  const int k_begin = lo + split * len;
  const int k_end = min(pos + 1, k_begin + len);
  const int n_tiles = k_end > k_begin ? (k_end - k_begin + KT - 1) / KT : 0;
  const int* table = block_table + static_cast<size_t>(ck_request(row_request[row])) * max_blocks;
  const size_t kv_row = static_cast<size_t>(n_kv_heads) * HD;

  bf16* my = KV + static_cast<size_t>(warp) * STAGES * 2 * TILE_ELEMS;
  // When the block's key range starts on a multiple of 16 (always, unless a window moves it) and pages hold at
  // least 16 keys, every 16 keys of a tile lie in one page: one table lookup serves 16 key rows.
  const bool by_halves = (k_begin & 15) == 0 && page_shift >= 4;
  // The pages of this warp's first tiles, one lookup per lane, all on their way at once: lane l holds the page of half
  // l % HALVES of the warp's tile l / HALVES. A tile's copies then start without a lookup of their own in front of them.
  constexpr int HALVES = KT / 16, AHEAD_TILES = 32 / HALVES;
  int my_page = 0;
  if (by_halves) {
    const int kb = k_begin + ((lane / HALVES) * DT_WARPS + warp) * KT + (lane % HALVES) * 16;
    if (kb < k_end) my_page = ck_page(table, kb >> page_shift, max_blocks);
  }
  auto load_tile = [&](int i, int stage) {          // this warp's i-th tile: block tile i * DT_WARPS + warp
    const int key0 = k_begin + (i * DT_WARPS + warp) * KT;
    bf16* kd = my + static_cast<size_t>(stage) * 2 * TILE_ELEMS;
    bf16* vd = kd + TILE_ELEMS;
    if (by_halves) {
#pragma unroll
      for (int hf = 0; hf < KT / 16; ++hf) {
        const int kb = key0 + hf * 16;
        size_t slot0 = 0;
        if (i < AHEAD_TILES) {
          const int page = __shfl_sync(0xffffffffu, my_page, i * HALVES + hf);
          slot0 = (static_cast<size_t>(page) << page_shift) + (kb & page_mask);
        } else if (kb < k_end) {
          slot0 = (static_cast<size_t>(ck_page(table, kb >> page_shift, max_blocks)) << page_shift) + (kb & page_mask);
        }
#pragma unroll
        for (int c = lane; c < 16 * CH; c += 32) {
          const int r = c / CH, ch = c % CH;
          const bool ok = kb + r < k_end;
          const size_t off = ok ? (slot0 + r) * kv_row + static_cast<size_t>(kvh) * HD + ch * 8 : 0;
          dt_cp_async16(kd + (hf * 16 + r) * LD + ch * 8, k_cache + off, ok);
          dt_cp_async16(vd + (hf * 16 + r) * LD + ch * 8, v_cache + off, ok);
        }
      }
      return;
    }
#pragma unroll
    for (int c = lane; c < KT * CH; c += 32) {
      const int r = c / CH, ch = c % CH;
      const int key = key0 + r;
      const bool ok = key < k_end;
      size_t off = 0;
      if (ok) {
        const size_t slot = (static_cast<size_t>(ck_page(table, key >> page_shift, max_blocks)) << page_shift) + (key & page_mask);
        off = slot * kv_row + static_cast<size_t>(kvh) * HD + ch * 8;
      }
      dt_cp_async16(kd + r * LD + ch * 8, k_cache + off, ok);
      dt_cp_async16(vd + r * LD + ch * 8, v_cache + off, ok);
    }
  };
  const int my_tiles = n_tiles > warp ? (n_tiles - warp + DT_WARPS - 1) / DT_WARPS : 0;
  // Keys and values of earlier steps do not depend on the kernel before this one (the step's positions and block
  // tables were uploaded before the step): their first tiles are requested before the wait for that kernel. Only
  // the tile that holds the newest key, which that kernel has just written, waits.
  unsigned deferred = 0;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < my_tiles) {
      if (k_begin + (s * DT_WARPS + warp + 1) * KT <= pos) load_tile(s, s);
      else deferred |= 1u << s;
    }
    asm volatile("cp.async.commit_group;\n" ::);
  }
  pdl_wait();
  pdl_trigger();
  if (deferred) {
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s)
      if (deferred & (1u << s)) load_tile(s, s);
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 0;\n" ::);      // the groups of the loop below count from here
  }
  // the group's query heads as the rows of one 16-row tile (rows past the group are zero)
  for (int c = tid; c < 16 * CH; c += DT_THREADS) {
    const int r = c / CH, ch = c % CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < ng)
      v = *reinterpret_cast<const uint4*>(q + static_cast<size_t>(row) * q_stride + static_cast<size_t>(head0 + r) * HD + ch * 8);
    *reinterpret_cast<uint4*>(Qs + r * LD + ch * 8) = v;
  }
  __syncthreads();
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int c = ks * 16 + (lane >> 4) * 8;
    dt_ldmatrix_x4(qf[ks], Qs + r * LD + c);
  }


  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

  for (int i = 0; i < my_tiles; ++i) {
    const int stage = i % STAGES;
    if (i + STAGES - 1 < my_tiles) load_tile(i + STAGES - 1, (i + STAGES - 1) % STAGES);
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 1));
    __syncwarp();
    const bf16* kt = my + static_cast<size_t>(stage) * 2 * TILE_ELEMS;
    const bf16* vt = kt + TILE_ELEMS;
    const int key0 = k_begin + (i * DT_WARPS + warp) * KT;

    float s[KT / 8][4];
#pragma unroll
    for (int j = 0; j < KT / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int np = 0; np < KT / 16; ++np) {
        uint32_t kb[4];
        const int key = np * 16 + (lane & 7) + (lane >> 4) * 8;
        const int c = ks * 16 + ((lane >> 3) & 1) * 8;
        dt_ldmatrix_x4(kb, kt + key * LD + c);
        dt_mma(s[2 * np], qf[ks], kb[0], kb[1]);
        dt_mma(s[2 * np + 1], qf[ks], kb[2], kb[3]);
      }
    }
    // raw scores stay in s; the maximum is kept in scaled (base-2) units and the scale is folded into the exponent
    const bool edge = key0 + KT > k_end;
    if (edge) {
#pragma unroll
      for (int j = 0; j < KT / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (key0 + j * 8 + 2 * t + (e & 1) >= k_end) s[j][e] = -INFINITY;
      }
    }
    uint32_t pf[KT / 16][4];
    {                                                  // rows 0 to 7
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < KT / 8; ++j) mx = fmaxf(mx, fmaxf(s[j][0], s[j][1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[0], mx * scale_log2);          // finite: the first key of every tile is in range
      const float corr = dt_exp2(m_run[0] - m_new);
      m_run[0] = m_new;
      float ls = 0.0f;
#pragma unroll
      for (int j = 0; j < KT / 8; ++j) {
        const float p0 = dt_exp2(fmaf(s[j][0], scale_log2, -m_new)), p1 = dt_exp2(fmaf(s[j][1], scale_log2, -m_new));
        ls += p0 + p1;
        pf[j >> 1][(j & 1) * 2] = dt_pack(p0, p1);
      }
      ls += __shfl_xor_sync(0xffffffffu, ls, 1);
      ls += __shfl_xor_sync(0xffffffffu, ls, 2);
      l_run[0] = l_run[0] * corr + ls;
#pragma unroll
      for (int j = 0; j < HD / 8; ++j) { o[j][0] *= corr; o[j][1] *= corr; }
    }
    if (wide) {                                        // rows 8 to 15
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < KT / 8; ++j) mx = fmaxf(mx, fmaxf(s[j][2], s[j][3]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[1], mx * scale_log2);
      const float corr = dt_exp2(m_run[1] - m_new);
      m_run[1] = m_new;
      float ls = 0.0f;
#pragma unroll
      for (int j = 0; j < KT / 8; ++j) {
        const float p2 = dt_exp2(fmaf(s[j][2], scale_log2, -m_new)), p3 = dt_exp2(fmaf(s[j][3], scale_log2, -m_new));
        ls += p2 + p3;
        pf[j >> 1][(j & 1) * 2 + 1] = dt_pack(p2, p3);
      }
      ls += __shfl_xor_sync(0xffffffffu, ls, 1);
      ls += __shfl_xor_sync(0xffffffffu, ls, 2);
      l_run[1] = l_run[1] * corr + ls;
#pragma unroll
      for (int j = 0; j < HD / 8; ++j) { o[j][2] *= corr; o[j][3] *= corr; }
    } else {                                           // no query heads there: P is zero, O stays zero
#pragma unroll
      for (int j = 0; j < KT / 8; ++j) pf[j >> 1][(j & 1) * 2 + 1] = 0u;
    }
#pragma unroll
    for (int kk = 0; kk < KT / 16; ++kk) {
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        uint32_t vb[4];
        const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = dp * 16 + (lane >> 4) * 8;
        dt_ldmatrix_x4_trans(vb, vt + key * LD + c);
        dt_mma(o[2 * dp], pf[kk], vb[0], vb[1]);
        dt_mma(o[2 * dp + 1], pf[kk], vb[2], vb[3]);
      }
    }
    __syncwarp();        // the warp is done with this stage before a later prefetch overwrites it
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  __syncthreads();       // every warp has left the pipeline buffers: they become the merge area

  constexpr int REC = HD + 2;
  float* mine = merge + static_cast<size_t>(warp) * 16 * REC;
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) {
    const int d = j * 8 + 2 * t;
    mine[g * REC + d] = o[j][0];
    mine[g * REC + d + 1] = o[j][1];
    mine[(g + 8) * REC + d] = o[j][2];
    mine[(g + 8) * REC + d + 1] = o[j][3];
  }
  if (t == 0) {
    mine[g * REC + HD] = m_run[0];
    mine[g * REC + HD + 1] = l_run[0];
    mine[(g + 8) * REC + HD] = m_run[1];
    mine[(g + 8) * REC + HD + 1] = l_run[1];
  }
  __syncthreads();
  for (int idx = tid; idx < ng * HD; idx += DT_THREADS) {
    const int r = idx / HD, d = idx % HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DT_WARPS; ++w) mm = fmaxf(mm, merge[(w * 16 + r) * REC + HD]);
    float a = 0.0f, ll = 0.0f;
#pragma unroll
    for (int w = 0; w < DT_WARPS; ++w) {
      const float* src = merge + (w * 16 + r) * REC;
      const float c = mm == -INFINITY ? 0.0f : exp2f(src[HD] - mm);
      a += src[d] * c;
      ll += src[HD + 1] * c;
    }
    const int head = head0 + r;
    if (n_split == 1) {
      out[static_cast<size_t>(row) * out_stride + static_cast<size_t>(head) * HD + d] = __float2bfloat16_rn(a / ll);
    } else if (cluster_merge) {
      // the splits of one (row, KV head) are the blocks of one cluster: every block leaves its record in the
      // shared memory of the cluster's first block
      namespace cg = cooperative_groups;
      float* xbuf = reinterpret_cast<float*>(dt_smem + xbuf_offset);
      float* dst = cg::this_cluster().map_shared_rank(xbuf, 0) + (static_cast<size_t>(split) * 16 + r) * REC;
      dst[d] = a;
      if (d == 0) {
        dst[HD] = mm;
        dst[HD + 1] = ll;
      }
    } else {
      float* dst = part + ((static_cast<size_t>(row) * n_heads + head) * part_stride + split) * REC;
      dst[d] = a;
      if (d == 0) {
        dst[HD] = mm;
        dst[HD + 1] = ll;
      }
    }
  }
  if (plan != nullptr && n_split > 1) {
    // The block that finds all other parts of its (row, group chunk) done merges them, in the order of the parts,
    // whoever came last: the result does not depend on timing. Its own records are re-read like the others'.
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      int* counter = counters + row * (n_kv_heads * chunks) + ychunk;
      const int before = atomicAdd(counter, 1);
      s_last = before == n_split - 1;
      if (s_last) *counter = 0;               // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int idx = tid; idx < ng * HD; idx += DT_THREADS) {
      const int r = idx / HD, d = idx % HD;
      const float* rec = part + (static_cast<size_t>(row) * n_heads + head0 + r) * part_stride * REC;
      float mm = -INFINITY;
      for (int sp = 0; sp < n_split; ++sp) mm = fmaxf(mm, __ldcg(rec + sp * REC + HD));
      float a = 0.0f, ll = 0.0f;
      for (int sp = 0; sp < n_split; ++sp) {
        const float* src = rec + sp * REC;
        const float ms = __ldcg(src + HD);
        const float c = ms == -INFINITY ? 0.0f : exp2f(ms - mm);
        a += __ldcg(src + d) * c;
        ll += __ldcg(src + HD + 1) * c;
      }
      out[static_cast<size_t>(row) * out_stride + static_cast<size_t>(head0 + r) * HD + d] = __float2bfloat16_rn(a / ll);
    }
    return;
  }
  if (n_split > 1 && cluster_merge) {
    cooperative_groups::this_cluster().sync();       // every record has arrived (and is visible) in block 0
    if (split == 0) {
      const float* xbuf = reinterpret_cast<const float*>(dt_smem + xbuf_offset);
      for (int idx = tid; idx < ng * HD; idx += DT_THREADS) {
        const int r = idx / HD, d = idx % HD;
        float mm = -INFINITY;
        for (int sp = 0; sp < n_split; ++sp) mm = fmaxf(mm, xbuf[(sp * 16 + r) * REC + HD]);
        float a = 0.0f, ll = 0.0f;
        for (int sp = 0; sp < n_split; ++sp) {          // in split order, as attention_combine_kernel
          const float* src = xbuf + (sp * 16 + r) * REC;
          const float c = src[HD] == -INFINITY ? 0.0f : exp2f(src[HD] - mm);
          a += src[d] * c;
          ll += src[HD + 1] * c;
        }
        out[static_cast<size_t>(row) * out_stride + static_cast<size_t>(head0 + r) * HD + d] = __float2bfloat16_rn(a / ll);
      }
    }
  }
}

template <int HD, int STAGES, int KT, int W>
int launch_decode_tc(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table, int max_blocks,
                     const int* positions, const int* row_request, void* out, int out_stride, float* part, int rows,
                     int n_heads, int n_kv_heads, int page_shift, float scale, int window, int n_split,
                     const void* ahead, long long ahead_bytes, cudaStream_t stream, const int* plan = nullptr,
                     int* counters = nullptr, int unit_cap = 0, int part_stride = 0) {
  constexpr size_t pipe = static_cast<size_t>(16 + W * STAGES * 2 * KT) * (HD + 8) * sizeof(bf16);
  constexpr size_t mrg = static_cast<size_t>(W) * 16 * (HD + 2) * sizeof(float);
  constexpr size_t base = ((pipe > mrg ? pipe : mrg) + 15) & ~static_cast<size_t>(15);
  // Up to 8 splits can merge through the shared memory of a cluster's first block instead of scratch and a second
  // kernel. Measured on B200 (1B shapes, decode step at batch 8): clusters of 2 blocks 0.832 ms, of 4 0.881 ms, of 3
  // 0.903 ms; scratch and the merge kernel with 3 splits 0.883 ms, with 4 0.866 ms: clusters whose size is a power of
  // two place well, the others do not. So a caller that brings scratch gets the cluster for 2, 4 and 8 splits.
  const bool cluster = plan == nullptr && n_split > 1 && n_split <= 8 && (part == nullptr || (n_split & (n_split - 1)) == 0);
  const size_t smem = base + (cluster ? static_cast<size_t>(n_split) * 16 * (HD + 2) * sizeof(float) : 0);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_attention_tc_kernel<HD, STAGES, KT, W>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = smem;
  }
  const int group = n_heads / n_kv_heads;
  dim3 grid(n_split, n_kv_heads * ((group + 15) / 16), rows);
  if (plan != nullptr) grid = dim3(unit_cap, 1, 1);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(W * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (cluster) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = static_cast<unsigned>(n_split);
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  if (pdl_mode() >= 1) {          // the kernel requests its first tiles of old keys before it waits
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  int rc = static_cast<int>(cudaLaunchKernelEx(
      &cfg, decode_attention_tc_kernel<HD, STAGES, KT, W>, static_cast<const bf16*>(q), q_stride, static_cast<const bf16*>(kc),
      static_cast<const bf16*>(vc), block_table, max_blocks, positions, row_request, static_cast<bf16*>(out), out_stride,
      part, n_heads, n_kv_heads, page_shift, scale * 1.4426950408889634f, window, n_split, cluster ? 1 : 0,
      static_cast<int>(base), pdl_mode() >= 1 ? ahead : nullptr, pdl_mode() >= 1 ? ahead_bytes : 0ll, plan, counters,
      plan != nullptr ? part_stride : n_split));
  if (rc != 0 || n_split == 1 || cluster || plan != nullptr) return rc;
  dim3 cgrid(n_heads, rows);
  const int cthreads = HD <= 32 ? 32 : (HD <= 64 ? 64 : 128);
  return launch(attention_combine_kernel<bf16>, cgrid, dim3(cthreads), 0, stream, static_cast<const float*>(part),
                static_cast<bf16*>(out), out_stride, n_heads, HD, n_split);
}

}  // namespace dl

// Floats of scratch that `dl_paged_attention_decode` needs for n_split > 1.
DL_EXPORT long long dl_paged_attention_decode_scratch(int rows, int n_heads, int head_dim, int n_split) {
  return n_split <= 1 ? 0 : static_cast<long long>(rows) * n_heads * n_split * (head_dim + 2);
}

// q/out: rows with head h at column h * head_dim. k_cache, v_cache: [pages, page_size, kv_heads, head_dim],
// page_size a power of two. part: fp32 scratch of dl_paged_attention_decode_scratch floats (may be null when
// n_split == 1). Every row attends keys [lo, positions[row]] of its request.
DL_EXPORT int dl_paged_attention_decode(int dtype, const void* q, int q_stride, const void* k_cache,
                                        const void* v_cache, const int* block_table, int max_blocks,
                                        const int* positions, const int* row_request, void* out, int out_stride,
                                        float* part, int rows, int n_heads, int n_kv_heads, int head_dim,
                                        int page_size, float scale, int window, int n_split, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype == 0)
    return dl::launch_decode<float>(q, q_stride, k_cache, v_cache, block_table, max_blocks, positions, row_request, out,
                                    out_stride, part, rows, n_heads, n_kv_heads, head_dim, page_size, scale, window,
                                    n_split, stream);
  if (dtype == 1)
    return dl::launch_decode<dl::bf16>(q, q_stride, k_cache, v_cache, block_table, max_blocks, positions, row_request,
                                       out, out_stride, part, rows, n_heads, n_kv_heads, head_dim, page_size, scale,
                                       window, n_split, stream);
  return DL_ERR_UNSUPPORTED;
}

// Head size -> (stages, keys per tile, warps) of the tensor-core kernel. A block's pipeline is warps * stages *
// 2 * keys * (head_dim + 8) * 2 bytes of shared memory: about 110 KB each, two blocks to an SM.
#define DL_DECODE_TC_CASES                           \
  DL_CASE(16, 4, 32, 4);                             \
  DL_CASE(32, 4, 32, 4);                             \
  DL_CASE(48, 3, 32, 4);                             \
  DL_CASE(64, 3, 16, 8);                             \
  DL_CASE(80, 3, 32, 4);                             \
  DL_CASE(96, 3, 16, 4);                             \
  DL_CASE(112, 3, 16, 4);                            \
  DL_CASE(128, 3, 16, 4);

// The tensor-core variant: bfloat16, head_dim a multiple of 16 up to 128, q rows 16-byte aligned. Same
// arguments as dl_paged_attention_decode. Up to 8 splits are the blocks of a thread-block cluster and merge through
// distributed shared memory (no scratch is touched); more splits use the scratch and the merge kernel.
// ahead, ahead_bytes: memory that the kernel after this one will stream (weights), requested into L2 before this
// kernel waits for the one in front of it; null / 0: nothing.
DL_EXPORT int dl_paged_attention_decode_tc(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                           const int* block_table, int max_blocks, const int* positions,
                                           const int* row_request, void* out, int out_stride, float* part, int rows,
                                           int n_heads, int n_kv_heads, int head_dim, int page_size, float scale,
                                           int window, int n_split, const void* ahead, long long ahead_bytes,
                                           cudaStream_t stream) {
  if (rows <= 0) return 0;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  if ((1 << page_shift) != page_size || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_split < 1 || rows > 65535 ||
      (q_stride & 7) || !(scale > 0.0f) || (n_split > 8 && part == nullptr))   // without scratch, up to 8 splits merge in a cluster
    return DL_ERR_UNSUPPORTED;
#define DL_CASE(H, S, T, NW)                                                                                           \
  case H:                                                                                                             \
    return dl::launch_decode_tc<H, S, T, NW>(q, q_stride, k_cache, v_cache, block_table, max_blocks, positions,        \
                                          row_request, out, out_stride, part, rows, n_heads, n_kv_heads, page_shift,  \
                                          scale, window, n_split, ahead, ahead_bytes, stream)
  switch (head_dim) {
    DL_DECODE_TC_CASES
    default:
      return DL_ERR_UNSUPPORTED;
  }
#undef DL_CASE
}

// The same kernel with the keys of all rows dealt out by the host (the step's attention plan) instead of every row
// being cut into the same number of parts: plan = int32 [4 + 4 * units]: plan[0] = units, then per unit (row, KV head
// chunk, part, parts of its row); the grid has unit_cap blocks (a number that does not change from step to step, so
// that a CUDA graph can hold it), of which the first plan[0] work. A row's keys are cut into its `parts` (at most
// part_stride) like n_split cuts them above. Rows with several parts leave their records in `part`
// (rows * n_heads * part_stride * (head_dim + 2) floats) and the last block to finish a (row, chunk) merges them;
// counters: int32 [rows * KV head chunks], zero before the first launch (the kernel leaves them zero).
DL_EXPORT int dl_paged_attention_decode_planned(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                                const int* block_table, int max_blocks, const int* positions,
                                                const int* row_request, void* out, int out_stride, float* part,
                                                int rows, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                                float scale, int window, const int* plan, int* counters, int unit_cap,
                                                int part_stride, const void* ahead, long long ahead_bytes,
                                                cudaStream_t stream) {
  if (rows <= 0 || unit_cap <= 0) return 0;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  if ((1 << page_shift) != page_size || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || part_stride < 1 || rows > 65535 ||
      (q_stride & 7) || !(scale > 0.0f) || plan == nullptr || counters == nullptr || part == nullptr ||
      (reinterpret_cast<uintptr_t>(plan) & 15))
    return DL_ERR_UNSUPPORTED;
#define DL_CASE(H, S, T, NW)                                                                                           \
  case H:                                                                                                             \
    return dl::launch_decode_tc<H, S, T, NW>(q, q_stride, k_cache, v_cache, block_table, max_blocks, positions,        \
                                          row_request, out, out_stride, part, rows, n_heads, n_kv_heads, page_shift,  \
                                          scale, window, 2, ahead, ahead_bytes, stream, plan, counters, unit_cap,     \
                                          part_stride)
  switch (head_dim) {
    DL_DECODE_TC_CASES
    default:
      return DL_ERR_UNSUPPORTED;
  }
#undef DL_CASE
}

// Keys per tile of the tensor-core kernel for a head size (what a plan counts the keys in).
DL_EXPORT int dl_paged_attention_decode_tile(int head_dim) {
#define DL_CASE(H, S, T, NW) \
  case H:                    \
    return T
  switch (head_dim) {
    DL_DECODE_TC_CASES
    default:
      return 0;
  }
#undef DL_CASE
}

// ------------------------------------------------------------------------------------------------
// The entry point that allocates nothing (see dynalm_noalloc.h for who needs it and its rules).
// ------------------------------------------------------------------------------------------------
#include "dynalm_noalloc.h"

#include <mutex>

// Partial results of the split-KV kernel, for callers that have no scratch to give. In host code this
// name is only a handle for cudaGetSymbolAddress: it is not a device address and must never be passed
// to a kernel as one.
static __device__ __align__(256) float dl_noalloc_scratch[DL_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mutex;

// The device address of the array on the current device, looked up once per device.
int noalloc_scratch(float** ptr) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return DL_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), dl_noalloc_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_noalloc_ptr[dev] = p;
  }
  *ptr = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

DL_EXPORT int dl_paged_attention_decode_noalloc(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                                const int* block_table, int max_blocks, const int* positions,
                                                const int* row_request, void* out, int out_stride, int rows,
                                                int n_heads, int n_kv_heads, int head_dim, int page_size, float scale,
                                                int window, int n_split, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (n_split < 1 || n_heads <= 0 || head_dim <= 0) return DL_ERR_UNSUPPORTED;
  const long long need = dl_paged_attention_decode_scratch(rows, n_heads, head_dim, n_split);
  if (need > DL_NOALLOC_SCRATCH_FLOATS) return DL_ERR_NOALLOC_TOO_LARGE;
  float* part = nullptr;
  if (need > 0) {
    const int rc = noalloc_scratch(&part);
    if (rc != 0) return rc;
  }
  return dl_paged_attention_decode_tc(q, q_stride, k_cache, v_cache, block_table, max_blocks, positions, row_request,
                                      out, out_stride, part, rows, n_heads, n_kv_heads, head_dim, page_size, scale,
                                      window, n_split, nullptr, 0, stream);
}

DL_EXPORT const char* dl_noalloc_strerror(int code) {
  switch (code) {
    case 0:
      return "ok";
    case DL_ERR_NOALLOC_TOO_LARGE:
      return "the call needs more scratch than the library's built-in array holds (rows * n_heads * n_split * "
             "(head_dim + 2) floats, at most 1048576): lower n_split or pass fewer rows per call";
    case DL_ERR_UNSUPPORTED:
      return "the kernel does not take these sizes (bfloat16, head_dim a multiple of 16 up to 128, page size a "
             "power of two, 16-byte aligned q rows)";
    default:
      return cudaGetErrorString(static_cast<cudaError_t>(code));
  }
}
