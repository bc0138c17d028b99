// RMSNorm over the fp32 residual stream, fused with the residual add that precedes it and with
// the gather of the rows whose logits are wanted.
//
//   v   = x[src] + delta_scale * delta[src]        (delta optional; src = rows[r] or r)
//   x[src] = v                                     (when write_residual)
//   out[r] = v * (1 / sqrt(mean(v^2) + eps)) * w
//
// Formula: CpuDevice::rms_norm (dynacore/cpu/cpu_device.cpp:1179-1205); the reference sums
// squares in double, here the sum is a fixed-order fp32 tree over the block. The residual add is
// a separate op in the reference (dynalm/src/model/transformer.cpp:657,697).
#include "common.cuh"

namespace dl {

// delta may come in `parts` partial sums, `part_stride` elements apart (a split-K matrix product
// leaves them so); they are added in index order, so the result does not depend on timing.
template <typename TD>
__device__ __forceinline__ float delta_at(const TD* dr, int i, int parts, size_t part_stride) {
  float d = to_float(dr[i]);
  for (int p = 1; p < parts; ++p) d += to_float(dr[p * part_stride + i]);
  return d;
}

template <typename TO, typename TD>
__global__ void rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, float delta_scale,
                               const float* __restrict__ w, float eps, TO* __restrict__ out,
                               const int* __restrict__ rows, int width, int write_residual, int parts,
                               size_t part_stride) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  const size_t src = rows ? static_cast<size_t>(ck_row(rows[r])) : static_cast<size_t>(r);
  float* xr = x + src * width;
  const TD* dr = delta ? delta + src * width : nullptr;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = xr[i];
    if (dr) {
      v = fmaf(delta_scale, delta_at(dr, i, parts, part_stride), v);
      if (write_residual) xr[i] = v;
    }
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  TO* orow = out + static_cast<size_t>(r) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = xr[i];
    if (dr && !write_residual) v = fmaf(delta_scale, delta_at(dr, i, parts, part_stride), v);
    orow[i] = from_float<TO>(v * inv * w[i]);
  }
}

// The same computation with the row held in registers: one pass over global memory, 16-byte
// accesses, every load of a thread issued before its first use. For widths that are a multiple of 4
// and at most NV * 1024.
template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<bf16>(const bf16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                     __uint_as_float(u.y & 0xffff0000u));
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

constexpr int NORM_VEC_THREADS = 256;

template <typename TO, typename TD, int NV>
__global__ void __launch_bounds__(NORM_VEC_THREADS)
rmsnorm_vec_kernel(float* __restrict__ x, const TD* __restrict__ delta, float delta_scale,
                   const float* __restrict__ w, float eps, TO* __restrict__ out, const int* __restrict__ rows,
                   int width, int write_residual, int parts, size_t part_stride, int n_rows,
                   const void* __restrict__ ahead, long long ahead_bytes) {
  __shared__ float red[33];
  l2_prefetch_share(ahead, ahead_bytes);       // the grid may have more blocks than rows for this
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  if (r >= n_rows) return;
  const size_t src = rows ? static_cast<size_t>(ck_row(rows[r])) : static_cast<size_t>(r);
  float* xr = x + src * width;
  const TD* dr = delta ? delta + src * width : nullptr;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 v[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * NORM_VEC_THREADS + threadIdx.x) * 4;
    v[i] = c < width ? load4<float>(xr + c) : zero;
  }
  if (dr) {
    float4 d[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * NORM_VEC_THREADS + threadIdx.x) * 4;
      d[i] = c < width ? load4<TD>(dr + c) : zero;
    }
    // parts are added in index order; the loads of two parts are issued together, so a product left in many
    // parts costs half the round trips (four at a time cost the three-part case 1 % of a decode step)
    constexpr int PC = NV <= 4 ? 2 : 1;
    for (int p = 1; p < parts; p += PC) {
      float4 e[PC][NV];
#pragma unroll
      for (int q = 0; q < PC; ++q) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int c = (i * NORM_VEC_THREADS + threadIdx.x) * 4;
          e[q][i] = (p + q < parts && c < width) ? load4<TD>(dr + (p + q) * part_stride + c) : zero;
        }
      }
#pragma unroll
      for (int q = 0; q < PC; ++q) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          d[i].x += e[q][i].x; d[i].y += e[q][i].y; d[i].z += e[q][i].z; d[i].w += e[q][i].w;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      v[i].x = fmaf(delta_scale, d[i].x, v[i].x); v[i].y = fmaf(delta_scale, d[i].y, v[i].y);
      v[i].z = fmaf(delta_scale, d[i].z, v[i].z); v[i].w = fmaf(delta_scale, d[i].w, v[i].w);
      const int c = (i * NORM_VEC_THREADS + threadIdx.x) * 4;
      if (write_residual && c < width) store4<float>(xr + c, v[i]);
    }
  }
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
    ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(width) + eps);
  TO* orow = out + static_cast<size_t>(r) * width;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * NORM_VEC_THREADS + threadIdx.x) * 4;
    if (c < width) {
      const float4 g = load4<float>(w + c);
      store4<TO>(orow + c, make_float4(v[i].x * inv * g.x, v[i].y * inv * g.y, v[i].z * inv * g.z, v[i].w * inv * g.w));
    }
  }
}

// x += scale * delta, for a pending residual that no norm follows.
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ x, const TD* __restrict__ delta, float scale, size_t n,
                                    int parts, size_t part_stride) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) {
    float d = to_float(delta[i]);
    for (int p = 1; p < parts; ++p) d += to_float(delta[p * part_stride + i]);
    x[i] = fmaf(scale, d, x[i]);
  }
}

}  // namespace dl

// out_dtype / delta_dtype: 0 = float32, 1 = bfloat16. delta and rows may be null. delta_parts >= 1 partial
// sums of delta lie delta_part_stride elements apart.
DL_EXPORT int dl_rmsnorm(int out_dtype, int delta_dtype, float* x, const void* delta, float delta_scale,
                         const float* w, float eps, void* out, const int* rows, int n_rows, int width,
                         int write_residual, int delta_parts, long long delta_part_stride, const void* ahead,
                         long long ahead_bytes, cudaStream_t stream) {
  // ahead, ahead_bytes: memory that the kernel after this one will stream (its weights), or null: requested into L2
  // before this kernel waits for the one in front of it (only the vector kernel does)
  if (n_rows <= 0) return 0;
  if (width % 4 == 0 && width <= 8 * 4 * dl::NORM_VEC_THREADS &&
      (delta_part_stride % 4 == 0)) {
    const int nv = (width + 4 * dl::NORM_VEC_THREADS - 1) / (4 * dl::NORM_VEC_THREADS);
    int rc = 0;
    // with memory to request ahead the kernel starts early (it requests before its wait) and brings blocks for that
    const bool ahead_on = ahead != nullptr && ahead_bytes > 0 && dl::pdl_mode() >= 1;
    const bool early = ahead_on || dl::pdl_mode() == 1;
    const int blocks = ahead_on ? (n_rows > 64 ? n_rows : 64) : n_rows;
    if (!ahead_on) ahead_bytes = 0;
#define DL_VEC(TO, TD, NV)                                                                                         \
  rc = dl::launch_impl(early, dl::rmsnorm_vec_kernel<TO, TD, NV>, dim3(blocks), dim3(dl::NORM_VEC_THREADS), 0, stream, x,  \
                       static_cast<const TD*>(delta), delta_scale, w, eps, static_cast<TO*>(out), rows, width,          \
                       write_residual, delta_parts, static_cast<size_t>(delta_part_stride), n_rows, ahead, ahead_bytes)
#define DL_VEC_NV(TO, TD)                                   \
  do {                                                      \
    if (nv <= 1) DL_VEC(TO, TD, 1);                         \
    else if (nv <= 2) DL_VEC(TO, TD, 2);                    \
    else if (nv <= 4) DL_VEC(TO, TD, 4);                    \
    else DL_VEC(TO, TD, 8);                                 \
  } while (0)
    if (out_dtype == 0 && delta_dtype == 0) DL_VEC_NV(float, float);
    else if (out_dtype == 1 && delta_dtype == 1) DL_VEC_NV(dl::bf16, dl::bf16);
    else if (out_dtype == 1 && delta_dtype == 0) DL_VEC_NV(dl::bf16, float);
    else if (out_dtype == 0 && delta_dtype == 1) DL_VEC_NV(float, dl::bf16);
    else return DL_ERR_UNSUPPORTED;
#undef DL_VEC_NV
#undef DL_VEC
    return rc;
  }
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
#define DL_LAUNCH(TO, TD)                                                                            \
  dl::rmsnorm_kernel<TO, TD><<<n_rows, threads, 0, stream>>>(x, static_cast<const TD*>(delta), delta_scale, w, eps, \
                                                             static_cast<TO*>(out), rows, width, write_residual, \
                                                             delta_parts, static_cast<size_t>(delta_part_stride))
  if (out_dtype == 0 && delta_dtype == 0) DL_LAUNCH(float, float);
  else if (out_dtype == 1 && delta_dtype == 1) DL_LAUNCH(dl::bf16, dl::bf16);
  else if (out_dtype == 1 && delta_dtype == 0) DL_LAUNCH(dl::bf16, float);
  else if (out_dtype == 0 && delta_dtype == 1) DL_LAUNCH(float, dl::bf16);
  else return DL_ERR_UNSUPPORTED;
#undef DL_LAUNCH
  return dl::launch_status();
}

DL_EXPORT int dl_residual_add(int delta_dtype, float* x, const void* delta, float scale, long long n,
                              int delta_parts, long long delta_part_stride, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((n + threads - 1) / threads);
  if (delta_dtype == 0) dl::residual_add_kernel<float><<<blocks, threads, 0, stream>>>(x, static_cast<const float*>(delta), scale, static_cast<size_t>(n), delta_parts, static_cast<size_t>(delta_part_stride));
  else if (delta_dtype == 1) dl::residual_add_kernel<dl::bf16><<<blocks, threads, 0, stream>>>(x, static_cast<const dl::bf16*>(delta), scale, static_cast<size_t>(n), delta_parts, static_cast<size_t>(delta_part_stride));
  else return DL_ERR_UNSUPPORTED;
  return dl::launch_status();
}
