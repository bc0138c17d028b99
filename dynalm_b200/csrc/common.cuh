// Shared device helpers for the sm_100a kernels of dynalm_b200.
//
// Every kernel file exports plain C entry points (DL_EXPORT) that take raw device pointers,
// sizes and a stream, launch on that stream and return a cudaError_t as int. Nothing here
// allocates device memory; callers own every buffer.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define DL_EXPORT extern "C" __attribute__((visibility("default")))

// Return code for "this size is not supported by the kernel" (never a wrong result).
#define DL_ERR_UNSUPPORTED 10001

namespace dl {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `red` is shared memory of at least 33 floats. Every thread gets the result.
// The order of additions is fixed by the block shape, not by the data.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? red[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// 16-byte vector of 8 bf16 / 4 floats, for coalesced row traffic.
struct __align__(16) Vec16 {
  uint4 raw;
};

template <typename T> struct PerVec;
template <> struct PerVec<float> { static constexpr int n = 4; };
template <> struct PerVec<bf16> { static constexpr int n = 8; };

template <typename T>
__device__ __forceinline__ void unpack(const Vec16& v, float* out);
template <>
__device__ __forceinline__ void unpack<float>(const Vec16& v, float* out) {
  out[0] = __uint_as_float(v.raw.x);
  out[1] = __uint_as_float(v.raw.y);
  out[2] = __uint_as_float(v.raw.z);
  out[3] = __uint_as_float(v.raw.w);
}
template <>
__device__ __forceinline__ void unpack<bf16>(const Vec16& v, float* out) {
  const uint32_t w[4] = {v.raw.x, v.raw.y, v.raw.z, v.raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <typename T>
__device__ __forceinline__ Vec16 pack(const float* in);
template <>
__device__ __forceinline__ Vec16 pack<float>(const float* in) {
  Vec16 v;
  v.raw = make_uint4(__float_as_uint(in[0]), __float_as_uint(in[1]), __float_as_uint(in[2]), __float_as_uint(in[3]));
  return v;
}
template <>
__device__ __forceinline__ Vec16 pack<bf16>(const float* in) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 p = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&p);
  }
  Vec16 v;
  v.raw = make_uint4(w[0], w[1], w[2], w[3]);
  return v;
}

inline int launch_status() { return static_cast<int>(cudaGetLastError()); }

// Programmatic dependent launch. A kernel launched with the attribute may begin while the kernel before it on
// the stream is still running; it must call pdl_wait() before it reads anything an earlier kernel wrote and
// before it writes anything at all. pdl_trigger() lets the kernel after it begin likewise; the kernels here call
// it after their own wait, so that at most two kernels share the SMs (with the trigger first, a whole chain of
// waiting kernels held slots that the running kernel's later blocks needed). Kernels launched the ordinary way
// treat both as no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Asks for this block's share of [p, p + bytes) to be brought into L2: pieces of 16 KB dealt to the grid's blocks in
// turn, each requested by one thread with one bulk prefetch. Nothing waits for it. A kernel that was launched early
// (programmatic dependent launch) calls it before its wait with the weights that the kernel after it will stream:
// they cross the memory bus while the kernels in front are still running, and are read from L2 when their turn comes.
__device__ __forceinline__ void l2_prefetch_share(const void* p, long long bytes) {
  if (p == nullptr || bytes <= 0 || threadIdx.x != 0 || threadIdx.y != 0 || threadIdx.z != 0) return;
  constexpr long long PIECE = 16384;
  const long long blocks = static_cast<long long>(gridDim.x) * gridDim.y * gridDim.z;
  const long long me = (static_cast<long long>(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
  const char* base = static_cast<const char*>(p);
  for (long long off = me * PIECE; off < bytes; off += blocks * PIECE) {
    const long long left = bytes - off;
    const unsigned n = static_cast<unsigned>(left < PIECE ? (left & ~15ll) : PIECE);
    if (n > 0) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + off), "r"(n) : "memory");
  }
}

// DYNALM_PDL: 2 or unset = only the weight-streaming kernels (`launch_streaming`), which request their first
// weights before they wait; 1 = every kernel launched through `launch` too; 0 = none. Measured on B200, decode
// step at batch 8 inside the CUDA graph: 0.99 ms with 0, 1.00 ms with 1, 0.95 ms with 2.
inline int pdl_mode() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("DYNALM_PDL");
    v = (e != nullptr && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 2;
  }
  return v;
}

template <typename... KArgs, typename... Args>
inline int launch_impl(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = early ? 1 : 0;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}

template <typename... KArgs, typename... Args>
inline int launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  return launch_impl(pdl_mode() == 1, kernel, grid, block, smem, stream, args...);
}

// For kernels that have work to do before their wait (weights to request).
template <typename... KArgs, typename... Args>
inline int launch_streaming(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  return launch_impl(pdl_mode() >= 1, kernel, grid, block, smem, stream, args...);
}

}  // namespace dl

#include "check.cuh"
