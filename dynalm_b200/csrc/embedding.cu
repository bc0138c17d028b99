// Token embedding gather: out[i, :] = table[ids[i], :] * scale, written as the fp32 residual stream.
// Reference op: CpuDevice::embedding (dynacore/cpu/cpu_device.cpp:212-219), scale applied as in
// dynalm/src/model/transformer.cpp:576-577.
#include "common.cuh"

namespace dl {

template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                             int width, int vocab, float scale) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  int id = ck_token(ids[row], vocab);
  // The step function has already refused ids outside [0, vocab); clamping keeps a stray id
  // from reading outside the table.
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const T* src = table + static_cast<size_t>(id) * width;
  float* dst = out + static_cast<size_t>(row) * width;
  constexpr int V = PerVec<T>::n;
  if (width % V == 0) {
    const Vec16* s = reinterpret_cast<const Vec16*>(src);
    for (int i = threadIdx.x; i < width / V; i += blockDim.x) {
      float f[V];
      unpack<T>(s[i], f);
#pragma unroll
      for (int j = 0; j < V; j += 4) {
        float4 o = make_float4(f[j] * scale, f[j + 1] * scale, f[j + 2] * scale, f[j + 3] * scale);
        *reinterpret_cast<float4*>(dst + i * V + j) = o;
      }
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = to_float(src[i]) * scale;
  }
}

}  // namespace dl

// dtype: 0 = float32 table, 1 = bfloat16 table.
DL_EXPORT int dl_embed(int dtype, const void* table, const int* ids, float* out, int rows, int width, int vocab,
                       float scale, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == 0) {
    return dl::launch(dl::embed_kernel<float>, dim3(rows), dim3(threads), 0, stream, static_cast<const float*>(table), ids, out, width, vocab, scale);
  } else if (dtype == 1) {
    return dl::launch(dl::embed_kernel<dl::bf16>, dim3(rows), dim3(threads), 0, stream, static_cast<const dl::bf16*>(table), ids, out, width, vocab, scale);
  } else {
    return DL_ERR_UNSUPPORTED;
  }
  return dl::launch_status();
}
