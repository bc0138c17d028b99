// Paged causal attention, one thread block per (query row, head): the plain kernel.
//
// It serves the true 32-bit path and every shape the faster kernels refuse. A row at position
// `pos` of request r reads keys t in [lo, pos], lo = window > 0 ? max(0, pos - window + 1) : 0,
// through block_table[r]; query head h reads KV head h / (heads / kv_heads).
//   s_t = scale * q.k_t;  out = sum_t exp(s_t - max) v_t / sum_t exp(s_t - max)
// (dynacore/cpu/cpu_device.cpp:1309-1412,1717-1776). Keys are visited in chunks whose boundaries
// are multiples of CHUNK in absolute position, merged by the running (max, sum, acc) rule of the
// reference's split-K variant (:1782-1845). What a row computes therefore depends only on its own
// query, position and keys: not on the other rows of the batch nor on how the prompt was cut.
// Scores, softmax and the weighted sum are fp32.
#include "common.cuh"

namespace dl {

constexpr int ATT_THREADS = 256;
constexpr int ATT_CHUNK = 512;

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
paged_attention_generic_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                               const T* __restrict__ v_cache, const int* __restrict__ block_table,
                               int max_blocks, const int* __restrict__ positions,
                               const int* __restrict__ row_request, T* __restrict__ out, int out_stride,
                               int n_heads, int n_kv_heads, int head_dim, int page_size, float scale,
                               int window) {
  __shared__ float red[33];
  __shared__ float sq[256];                 // the query, fp32
  __shared__ float sp[ATT_CHUNK];           // scores, then probabilities, of one chunk
  __shared__ float part[ATT_THREADS];       // partial weighted sums, [group][dim]
  const int row = blockIdx.x, head = blockIdx.y;
  const int kvh = head / (n_heads / n_kv_heads);
  const int pos = positions[row];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int* table = block_table + static_cast<size_t>(ck_request(row_request[row])) * max_blocks;
  const int tid = threadIdx.x;

  const T* qrow = q + static_cast<size_t>(row) * q_stride + static_cast<size_t>(head) * head_dim;
  for (int d = tid; d < head_dim; d += ATT_THREADS) sq[d] = to_float(qrow[d]);
  __syncthreads();

  constexpr int V = PerVec<T>::n;
  const int groups = ATT_THREADS / head_dim;          // >= 1 since head_dim <= 256
  const int g = tid / head_dim, d = tid % head_dim;   // valid when g < groups
  const size_t kv_row = static_cast<size_t>(n_kv_heads) * head_dim;

  float m_run = -INFINITY, l_run = 0.0f, acc = 0.0f;  // acc: dim `tid` of the output, threads < head_dim
  for (int c0 = (lo / ATT_CHUNK) * ATT_CHUNK; c0 <= pos; c0 += ATT_CHUNK) {
    const int c1 = min(c0 + ATT_CHUNK, pos + 1);
    float m_loc = -INFINITY;
    for (int t = c0 + tid; t < c1; t += ATT_THREADS) {
      float s = -INFINITY;
      if (t >= lo) {
        const size_t slot = static_cast<size_t>(ck_page(table, t / page_size, max_blocks)) * page_size + t % page_size;
        const Vec16* kr = reinterpret_cast<const Vec16*>(k_cache + slot * kv_row + static_cast<size_t>(kvh) * head_dim);
        float dot = 0.0f;
        for (int i = 0; i < head_dim / V; ++i) {
          float f[V];
          unpack<T>(kr[i], f);
#pragma unroll
          for (int j = 0; j < V; ++j) dot = fmaf(sq[i * V + j], f[j], dot);
        }
        s = dot * scale;
      }
      sp[t - c0] = s;
      m_loc = fmaxf(m_loc, s);
    }
    const float m_chunk = block_max(m_loc, red);
    const float m_new = fmaxf(m_run, m_chunk);          // finite: the chunk holds at least key max(lo, c0)
    float l_loc = 0.0f;
    for (int t = c0 + tid; t < c1; t += ATT_THREADS) {
      const float p = expf(sp[t - c0] - m_new);         // exp(-inf) = 0 for keys before lo
      sp[t - c0] = p;
      l_loc += p;
    }
    const float l_chunk = block_sum(l_loc, red);        // also orders the writes of sp before the reads below
    const float corr = expf(m_run - m_new);             // 0 on the first chunk
    l_run = l_run * corr + l_chunk;
    m_run = m_new;

    float pv = 0.0f;
    if (g < groups) {
      const int t0 = max(c0, lo);
      for (int t = t0 + g; t < c1; t += groups) {
        const size_t slot = static_cast<size_t>(ck_page(table, t / page_size, max_blocks)) * page_size + t % page_size;
        pv = fmaf(sp[t - c0], to_float(v_cache[slot * kv_row + static_cast<size_t>(kvh) * head_dim + d]), pv);
      }
    }
    part[tid] = pv;
    __syncthreads();
    if (tid < head_dim) {
      float sum = 0.0f;
      for (int gg = 0; gg < groups; ++gg) sum += part[gg * head_dim + tid];
      acc = acc * corr + sum;
    }
    __syncthreads();
  }
  if (tid < head_dim) {
    T* orow = out + static_cast<size_t>(row) * out_stride + static_cast<size_t>(head) * head_dim;
    orow[tid] = from_float<T>(acc / l_run);
  }
}

}  // namespace dl

// q: rows of `q_stride` elements with head h at column h * head_dim; out likewise with out_stride.
// k_cache, v_cache: [pages, page_size, n_kv_heads, head_dim]. head_dim: a multiple of 16 up to 256.
DL_EXPORT int dl_paged_attention_generic(int dtype, const void* q, int q_stride, const void* k_cache,
                                         const void* v_cache, const int* block_table, int max_blocks,
                                         const int* positions, const int* row_request, void* out,
                                         int out_stride, int rows, int n_heads, int n_kv_heads, int head_dim,
                                         int page_size, float scale, int window, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (head_dim % 16 != 0 || head_dim > 256 || head_dim <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 ||
      page_size <= 0 || n_heads > 65535)
    return DL_ERR_UNSUPPORTED;
  dim3 grid(rows, n_heads);
#define DL_LAUNCH(T)                                                                                          \
  dl::paged_attention_generic_kernel<T><<<grid, dl::ATT_THREADS, 0, stream>>>(                                 \
      static_cast<const T*>(q), q_stride, static_cast<const T*>(k_cache), static_cast<const T*>(v_cache),     \
      block_table, max_blocks, positions, row_request, static_cast<T*>(out), out_stride, n_heads, n_kv_heads, \
      head_dim, page_size, scale, window)
  if (dtype == 0) DL_LAUNCH(float);
  else if (dtype == 1) DL_LAUNCH(dl::bf16);
  else return DL_ERR_UNSUPPORTED;
#undef DL_LAUNCH
  return dl::launch_status();
}
