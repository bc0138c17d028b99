// Rotary position encoding of queries and keys, fused with the write of keys and values into the
// paged cache.
//
// Rotation (half-split pairs, the Hugging Face layout): for pair i < rot/2 of every head,
//   theta = float(pos) * pos_scale * inv_freq[i]
//   a' = a cos(theta) - b sin(theta),  b' = a sin(theta) + b cos(theta),  (a, b) = (x[i], x[i + rot/2])
// as CpuDevice::rope (dynacore/cpu/cpu_device.cpp:1228-1262); inv_freq comes from the host already
// divided by the llama3 factors. Angles, sine and cosine are fp32 with full-range reduction.
// Keys are cached rotated (dynalm/src/model/transformer.cpp:630-637). Cache layout is slot-major:
// [page][slot][kv_head][dim] (dynacore/include/dynacore/attention/paged_kv.h:16-25), the page of
// position p of request r being block_table[r][p / page_size].
#include "common.cuh"

namespace dl {

template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                                  const int* __restrict__ row_request, const int* __restrict__ block_table,
                                  int max_blocks, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                  const float* __restrict__ inv_freq, int rot, float pos_scale, int n_heads,
                                  int n_kv_heads, int head_dim, int page_size, int write_cache) {
  extern __shared__ float cs[];  // cos[rot/2], sin[rot/2]
  const int row = blockIdx.x;
  const int pos = positions[row];
  const int half = inv_freq ? rot / 2 : 0;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float theta = static_cast<float>(pos) * pos_scale * inv_freq[i];
    float s, c;
    sincosf(theta, &s, &c);
    cs[i] = c;
    cs[half + i] = s;
  }
  __syncthreads();

  T* base = qkv + static_cast<size_t>(row) * row_stride;
  T* kdst = nullptr;
  T* vdst = nullptr;
  if (write_cache) {
    const int req = ck_request(row_request[row]);
    const int page = ck_page_store(block_table + static_cast<size_t>(req) * max_blocks, pos / page_size, max_blocks);
    if (page < 0) {
      write_cache = 0;          // only a checked build comes here: the row's keys and values are not stored
    } else {
      const size_t slot = static_cast<size_t>(page) * page_size + pos % page_size;
      kdst = k_cache + slot * n_kv_heads * head_dim;
      vdst = v_cache + slot * n_kv_heads * head_dim;
    }
  }
  const int q_width = n_heads * head_dim, kv_width = n_kv_heads * head_dim;

  // rotated pairs of q and k heads; the k pairs go to the cache from the thread that made them
  const int rot_heads = write_cache ? n_heads + n_kv_heads : n_heads;
  for (int idx = threadIdx.x; idx < rot_heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    T* hx = base + static_cast<size_t>(h) * head_dim;  // k heads follow q heads in the row
    const float a = to_float(hx[i]), b = to_float(hx[i + half]);
    const float c = cs[i], s = cs[half + i];
    const T ra = from_float<T>(a * c - b * s), rb = from_float<T>(a * s + b * c);
    if (h < n_heads) {
      hx[i] = ra;
      hx[i + half] = rb;
    } else {
      T* kd = kdst + static_cast<size_t>(h - n_heads) * head_dim;
      kd[i] = ra;
      kd[i + half] = rb;
    }
  }
  if (!write_cache) return;
  // unrotated tail of each key head
  const int tail = head_dim - 2 * half;
  for (int idx = threadIdx.x; idx < n_kv_heads * tail; idx += blockDim.x) {
    const int h = idx / tail, d = 2 * half + idx % tail;
    kdst[static_cast<size_t>(h) * head_dim + d] = base[q_width + static_cast<size_t>(h) * head_dim + d];
  }
  for (int idx = threadIdx.x; idx < kv_width; idx += blockDim.x) vdst[idx] = base[q_width + kv_width + idx];
}

// The same with 16-byte accesses: rot / 2, head_dim and row_stride are multiples of the vector length.
template <typename T>
__global__ void rope_cache_vec_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                                      const int* __restrict__ row_request, const int* __restrict__ block_table,
                                      int max_blocks, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                      const float* __restrict__ inv_freq, int rot, float pos_scale, int n_heads,
                                      int n_kv_heads, int head_dim, int page_size, int write_cache) {
  constexpr int V = PerVec<T>::n;
  extern __shared__ float cs[];  // cos[rot/2], sin[rot/2]
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const int pos = positions[row];
  const int half = inv_freq ? rot / 2 : 0;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float theta = static_cast<float>(pos) * pos_scale * inv_freq[i];
    float s, c;
    sincosf(theta, &s, &c);
    cs[i] = c;
    cs[half + i] = s;
  }
  __syncthreads();
  T* base = qkv + static_cast<size_t>(row) * row_stride;
  T* kdst = nullptr;
  T* vdst = nullptr;
  if (write_cache) {
    const int req = ck_request(row_request[row]);
    const int page = ck_page_store(block_table + static_cast<size_t>(req) * max_blocks, pos / page_size, max_blocks);
    if (page < 0) {
      write_cache = 0;          // only a checked build comes here: the row's keys and values are not stored
    } else {
      const size_t slot = static_cast<size_t>(page) * page_size + pos % page_size;
      kdst = k_cache + slot * n_kv_heads * head_dim;
      vdst = v_cache + slot * n_kv_heads * head_dim;
    }
  }
  const int q_width = n_heads * head_dim, kv_width = n_kv_heads * head_dim;
  const int hc = half / V;                        // vector pairs per head
  const int rot_heads = write_cache ? n_heads + n_kv_heads : n_heads;
  for (int idx = threadIdx.x; idx < rot_heads * hc; idx += blockDim.x) {
    const int h = idx / hc, ci = idx % hc;
    T* hx = base + static_cast<size_t>(h) * head_dim + ci * V;
    float a[V], b[V], ra[V], rb[V];
    unpack<T>(*reinterpret_cast<const Vec16*>(hx), a);
    unpack<T>(*reinterpret_cast<const Vec16*>(hx + half), b);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float c = cs[ci * V + j], sn = cs[half + ci * V + j];
      ra[j] = a[j] * c - b[j] * sn;
      rb[j] = a[j] * sn + b[j] * c;
    }
    T* dst = h < n_heads ? hx : kdst + static_cast<size_t>(h - n_heads) * head_dim + ci * V;
    *reinterpret_cast<Vec16*>(dst) = pack<T>(ra);
    *reinterpret_cast<Vec16*>(dst + half) = pack<T>(rb);
  }
  if (!write_cache) return;
  const int tail = (head_dim - 2 * half) / V;     // unrotated vectors of each key head
  for (int idx = threadIdx.x; idx < n_kv_heads * tail; idx += blockDim.x) {
    const int h = idx / tail, d = 2 * half + (idx % tail) * V;
    *reinterpret_cast<Vec16*>(kdst + static_cast<size_t>(h) * head_dim + d) =
        *reinterpret_cast<const Vec16*>(base + q_width + static_cast<size_t>(h) * head_dim + d);
  }
  for (int idx = threadIdx.x; idx < kv_width / V; idx += blockDim.x)
    *reinterpret_cast<Vec16*>(vdst + idx * V) = *reinterpret_cast<const Vec16*>(base + q_width + kv_width + idx * V);
}

// (cos, sin) of every rotary pair of every row of a step: out[row * half + i] = sincos(float(pos) * pos_scale *
// inv_freq[i]), the values the kernels above compute for themselves. A step computes them once for all layers
// whose projection kernel rotates in its epilogue (gemm_tcgen05.cu).
__global__ void rope_angles_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, int half,
                                   float pos_scale, int rows, float2* __restrict__ out) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * half) return;
  const int row = idx / half, i = idx % half;
  const float theta = static_cast<float>(positions[row]) * pos_scale * inv_freq[i];
  float s, c;
  sincosf(theta, &s, &c);
  out[idx] = make_float2(c, s);
}

}  // namespace dl

DL_EXPORT int dl_rope_angles(const int* positions, const float* inv_freq, int half, float pos_scale, int rows, void* out,
                             cudaStream_t stream) {
  if (rows <= 0 || half <= 0) return 0;
  const long long n = static_cast<long long>(rows) * half;
  if (n > (1ll << 30)) return DL_ERR_UNSUPPORTED;
  dl::rope_angles_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(positions, inv_freq, half, pos_scale,
                                                                                     rows, static_cast<float2*>(out));
  return dl::launch_status();
}

// qkv: [rows, row_stride] with q | k | v side by side; q is rotated in place, k is rotated on its way
// into the cache (the k columns of qkv are left unrotated), v is copied. inv_freq may be null (no
// rotation). write_cache = 0 rotates q only (a layer that reads another layer's cache).
DL_EXPORT int dl_rope_cache_write(int dtype, void* qkv, int row_stride, const int* positions,
                                  const int* row_request, const int* block_table, int max_blocks, void* k_cache,
                                  void* v_cache, const float* inv_freq, int rot, float pos_scale, int rows,
                                  int n_heads, int n_kv_heads, int head_dim, int page_size, int write_cache,
                                  cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (rot < 0 || rot > head_dim || (rot & 1)) return DL_ERR_UNSUPPORTED;
  const int threads = 256;
  const size_t smem = static_cast<size_t>(rot) * sizeof(float);
  if (smem > 48 * 1024) return DL_ERR_UNSUPPORTED;
  const int vec = dtype == 0 ? 4 : 8;
  const int half = inv_freq ? rot / 2 : 0;
  if ((dtype == 0 || dtype == 1) && half % vec == 0 && head_dim % vec == 0 && row_stride % vec == 0 &&
      (reinterpret_cast<uintptr_t>(qkv) & 15) == 0) {
#define DL_LAUNCH_VEC(T)                                                                                            \
  dl::launch(dl::rope_cache_vec_kernel<T>, dim3(rows), dim3(threads), smem, stream, static_cast<T*>(qkv), row_stride, \
             positions, row_request, block_table, max_blocks, static_cast<T*>(k_cache), static_cast<T*>(v_cache),   \
             inv_freq, rot, pos_scale, n_heads, n_kv_heads, head_dim, page_size, write_cache)
    if (dtype == 0) return DL_LAUNCH_VEC(float);
    return DL_LAUNCH_VEC(dl::bf16);
#undef DL_LAUNCH_VEC
  }
#define DL_LAUNCH(T)                                                                                              \
  dl::rope_cache_kernel<T><<<rows, threads, smem, stream>>>(static_cast<T*>(qkv), row_stride, positions, row_request, \
                                                            block_table, max_blocks, static_cast<T*>(k_cache),    \
                                                            static_cast<T*>(v_cache), inv_freq, rot, pos_scale,   \
                                                            n_heads, n_kv_heads, head_dim, page_size, write_cache)
  if (dtype == 0) DL_LAUNCH(float);
  else if (dtype == 1) DL_LAUNCH(dl::bf16);
  else return DL_ERR_UNSUPPORTED;
#undef DL_LAUNCH
  return dl::launch_status();
}
