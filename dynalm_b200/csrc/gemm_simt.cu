// y = x W^T (+ bias): the plain matrix product, fp32 accumulation on the CUDA cores.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no reduced-precision mode)
// and the fallback for shapes the tensor-core kernels refuse. Every output element is one thread's
// running fused multiply-add over k = 0 .. K-1 in order, so its value does not depend on the number
// of rows in the call nor on where the row sits (the reference's matmul accumulates in fp32 too,
// dynacore/cpu/generic/kernels_generic.cpp:23-34). x: [M, K] (row stride ldx), W: [N, K] row-major,
// y: [M, N] (row stride ldy), bias: fp32 [N] or null.
#include "common.cuh"

namespace dl {

constexpr int GM = 64, GN = 64, GK = 16;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TX* __restrict__ x, int ldx, const TW* __restrict__ w, const float* __restrict__ bias,
                 TO* __restrict__ y, int ldy, int M, int N, int K, float out_scale) {
  __shared__ float xs[GK][GM + 4];
  __shared__ float ws[GK][GN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * GM, n0 = blockIdx.x * GN;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += GK) {
    // 64 x 16 tile of each operand: 1024 elements, 4 per thread
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      const int r = e / GK, c = e % GK;
      const int gk = k0 + c;
      float xv = 0.0f, wv = 0.0f;
      if (gk < K) {
        if (m0 + r < M) xv = to_float(x[static_cast<size_t>(m0 + r) * ldx + gk]);
        if (n0 + r < N) wv = to_float(w[static_cast<size_t>(n0 + r) * K + gk]);
      }
      xs[c][r] = xv;
      ws[c][r] = wv;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[k][tn + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + tm + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tn + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      y[static_cast<size_t>(m) * ldy + n] = from_float<TO>(v * out_scale);
    }
  }
}

}  // namespace dl

// in_dtype (x and W) / out_dtype: 0 = float32, 1 = bfloat16.
DL_EXPORT int dl_gemm_simt(int in_dtype, int out_dtype, const void* x, int ldx, const void* w, const float* bias,
                           void* y, int ldy, int M, int N, int K, float out_scale, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return DL_ERR_UNSUPPORTED;
  dim3 grid((N + dl::GN - 1) / dl::GN, (M + dl::GM - 1) / dl::GM);
  if (grid.y > 65535) return DL_ERR_UNSUPPORTED;
#define DL_LAUNCH(TI, TO)                                                                                   \
  dl::gemm_simt_kernel<TI, TI, TO><<<grid, 256, 0, stream>>>(static_cast<const TI*>(x), ldx,                \
                                                             static_cast<const TI*>(w), bias,               \
                                                             static_cast<TO*>(y), ldy, M, N, K, out_scale)
  if (in_dtype == 0 && out_dtype == 0) DL_LAUNCH(float, float);
  else if (in_dtype == 1 && out_dtype == 1) DL_LAUNCH(dl::bf16, dl::bf16);
  else if (in_dtype == 1 && out_dtype == 0) DL_LAUNCH(dl::bf16, float);
  else return DL_ERR_UNSUPPORTED;
#undef DL_LAUNCH
  return dl::launch_status();
}
