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
  const size_t src = rows ? static_cast<size_t>(rows[r]) : static_cast<size_t>(r);
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
                         int write_residual, int delta_parts, long long delta_part_stride, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
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
