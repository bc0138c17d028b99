// Gated activation: out[t, j] = silu(gu[t, j]) * gu[t, inner + j], gu = [gate | up] side by side.
// silu(x) = x * sigmoid(x) (dynacore/cpu/cpu_device.cpp:117-123; CpuDevice::act_mul :1912-1929).
// The math is fp32 whatever the storage type.
#include "common.cuh"

namespace dl {

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int rows, int inner) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t total = static_cast<size_t>(rows) * inner;
  if (idx >= total) return;
  const size_t t = idx / inner, j = idx % inner;
  const float g = to_float(gu[t * 2 * inner + j]);
  const float u = to_float(gu[t * 2 * inner + inner + j]);
  const float s = g / (1.0f + expf(-g));
  out[idx] = from_float<T>(s * u);
}

// 16 bytes per access; inner is a multiple of the vector length and rows of gu are 16-byte aligned.
template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int rows, int inner) {
  constexpr int V = PerVec<T>::n;
  const int per_row = inner / V;
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(rows) * per_row) return;
  const size_t t = idx / per_row, c = (idx % per_row) * V;
  float g[V], u[V], o[V];
  unpack<T>(*reinterpret_cast<const Vec16*>(gu + t * 2 * inner + c), g);
  unpack<T>(*reinterpret_cast<const Vec16*>(gu + t * 2 * inner + inner + c), u);
#pragma unroll
  for (int j = 0; j < V; ++j) o[j] = g[j] / (1.0f + expf(-g[j])) * u[j];
  *reinterpret_cast<Vec16*>(out + t * inner + c) = pack<T>(o);
}

}  // namespace dl

DL_EXPORT int dl_silu_mul(int dtype, const void* gu, void* out, int rows, int inner, cudaStream_t stream) {
  if (rows <= 0 || inner <= 0) return 0;
  const int threads = 256;
  const int vec = dtype == 0 ? 4 : 8;
  if ((dtype == 0 || dtype == 1) && inner % vec == 0 && (reinterpret_cast<uintptr_t>(gu) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    const size_t n = static_cast<size_t>(rows) * (inner / vec);
    const unsigned blocks = static_cast<unsigned>((n + threads - 1) / threads);
    if (dtype == 0) dl::silu_mul_vec_kernel<float><<<blocks, threads, 0, stream>>>(static_cast<const float*>(gu), static_cast<float*>(out), rows, inner);
    else dl::silu_mul_vec_kernel<dl::bf16><<<blocks, threads, 0, stream>>>(static_cast<const dl::bf16*>(gu), static_cast<dl::bf16*>(out), rows, inner);
    return dl::launch_status();
  }
  const size_t total = static_cast<size_t>(rows) * inner;
  const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
  if (dtype == 0) dl::silu_mul_kernel<float><<<blocks, threads, 0, stream>>>(static_cast<const float*>(gu), static_cast<float*>(out), rows, inner);
  else if (dtype == 1) dl::silu_mul_kernel<dl::bf16><<<blocks, threads, 0, stream>>>(static_cast<const dl::bf16*>(gu), static_cast<dl::bf16*>(out), rows, inner);
  else return DL_ERR_UNSUPPORTED;
  return dl::launch_status();
}
