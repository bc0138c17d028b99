// Token selection on the device: greedy argmax and temperature sampling over fp32 logits rows.
//
// Greedy: the index of the largest logit, ties to the lowest id (sample_greedy,
// dynalm/src/sampling/sampler.cpp:31-38). Temperature: p_i = exp((l_i - max) / T), the total summed in
// double, u * total walked down the ids in order until it goes negative, the last id on rounding
// (Sampler::distribution and ::draw, :120-137,209-220). The uniform u comes from the host, where the
// per-request xoshiro256** generator lives. The reference samples on the host from downloaded logits;
// here only the chosen ids leave the device.
#include <cooperative_groups.h>

#include "common.cuh"

namespace dl {

constexpr int SAMPLE_THREADS = 1024;

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int ld, int vocab, int* __restrict__ out,
              const int* __restrict__ status_src, int* __restrict__ status_dst) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  if (status_dst != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *status_dst = *status_src;
  const float* row = logits + static_cast<size_t>(blockIdx.x) * ld;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (v > best) { best = v; idx = i; }   // ascending i per thread: the first maximum is kept
  }
  auto better = [](float v, int i, float bv_, int bi_) { return v > bv_ || (v == bv_ && i < bi_); };
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
  __syncthreads();
  if (warp == 0) {
    best = lane < (blockDim.x >> 5) ? bv[lane] : -INFINITY;
    idx = lane < (blockDim.x >> 5) ? bi[lane] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
    }
    if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;   // NaN-only rows give 0, as the reference
  }
}

// Large vocabularies: ARGMAX_PARTS blocks per row each scan a contiguous slice and leave (value, index);
// a second small kernel picks among them. Ties still go to the lowest index: slices are in index
// order and the comparison prefers the lower index on equal values.
constexpr int ARGMAX_PARTS = 32;

__global__ void __launch_bounds__(256)
argmax_part_kernel(const float* __restrict__ logits, int ld, int vocab, float* __restrict__ pv, int* __restrict__ pi) {
  __shared__ float bv[8];
  __shared__ int bi[8];
  const int r = blockIdx.y, part = blockIdx.x;
  const int per = ((vocab + ARGMAX_PARTS - 1) / ARGMAX_PARTS + 3) & ~3;      // slices start at multiples of 4
  const int b = min(vocab, part * per), e = min(vocab, b + per);
  const float* row = logits + static_cast<size_t>(r) * ld;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  int i0 = b;
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    // 16 bytes a load, a thread's loads of the slice all issued before the first comparison; within a thread the
    // indices still rise, so the strict comparison keeps the lowest index among equal values
    const int e4 = b + ((e - b) & ~3);
#pragma unroll 4
    for (int i = b + threadIdx.x * 4; i < e4; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + i);
      if (v.x > best) { best = v.x; idx = i; }
      if (v.y > best) { best = v.y; idx = i + 1; }
      if (v.z > best) { best = v.z; idx = i + 2; }
      if (v.w > best) { best = v.w; idx = i + 3; }
    }
    i0 = e4;
  }
  for (int i = i0 + threadIdx.x; i < e; i += blockDim.x) {
    const float v = row[i];
    if (v > best) { best = v; idx = i; }
  }
  auto better = [](float v, int i, float bv_, int bi_) { return v > bv_ || (v == bv_ && i < bi_); };
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (better(bv[w], bi[w], best, idx)) { best = bv[w]; idx = bi[w]; }
    pv[r * ARGMAX_PARTS + part] = best;
    pi[r * ARGMAX_PARTS + part] = idx;
  }
}

__global__ void argmax_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int* __restrict__ out,
                                    const int* __restrict__ status_src, int* __restrict__ status_dst) {
  const int r = blockIdx.x, lane = threadIdx.x;     // 32 threads
  if (status_dst != nullptr && r == 0 && lane == 0) *status_dst = *status_src;
  float best = pv[r * ARGMAX_PARTS + lane];
  int idx = pi[r * ARGMAX_PARTS + lane];
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
  }
  if (lane == 0) out[r] = idx == 0x7fffffff ? 0 : idx;
}

// The same choice among any number of partial results per row (pv, pi: [rows][parts]): one block per row.
__global__ void __launch_bounds__(256)
argmax_of_parts_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int parts, int* __restrict__ out,
                       const int* __restrict__ status_src, int* __restrict__ status_dst) {
  __shared__ float bv[8];
  __shared__ int bi[8];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  if (status_dst != nullptr && r == 0 && threadIdx.x == 0) *status_dst = *status_src;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int p = threadIdx.x; p < parts; p += 256) {
    const float v = pv[static_cast<size_t>(r) * parts + p];
    const int i = pi[static_cast<size_t>(r) * parts + p];
    if (v > best || (v == best && i < idx)) { best = v; idx = i; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
  }
  if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int wv = 1; wv < 8; ++wv)
      if (bv[wv] > best || (bv[wv] == best && bi[wv] < idx)) { best = bv[wv]; idx = bi[wv]; }
    out[r] = idx == 0x7fffffff ? 0 : idx;
  }
}

// A thread-block cluster per row (one block for a small vocabulary, up to eight for a large one). Thread
// g = block's rank * SAMPLE_THREADS + thread owns the ids [g * per, (g + 1) * per), so that runs, threads and blocks
// are all in id order. Three passes over the row, each thread over its own run (the second and third find it in the
// caches): the largest logit (block tree, then the blocks' results read from one another's shared memory); the mass
// of each run in double and its place in the running total (a scan over the block, then the blocks' totals read
// the same way); the walk down the one run in which u * total falls. That run is the last whose start is at or
// below u * total; the walk inside it subtracts id by id as the reference does, and where rounding leaves it
// unfinished at the run's end it goes on to the next id with any mass, else the last id.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_temperature_kernel(const float* __restrict__ logits, int ld, int vocab, int per,
                          const float* __restrict__ temperature, const double* __restrict__ uniform,
                          int* __restrict__ out) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float red[33];
  __shared__ float block_m;          // read by the other blocks of the cluster
  __shared__ double block_total;     // likewise
  __shared__ double warp_before[32];
  __shared__ int winner;             // the first block's copy is the cluster's
  const int nblocks = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  const int r = blockIdx.x / nblocks;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* row = logits + static_cast<size_t>(r) * ld;
  const float inv_t = 1.0f / temperature[r];
  const int g = rank * SAMPLE_THREADS + static_cast<int>(threadIdx.x);
  const int b = static_cast<int>(min(static_cast<long long>(vocab), static_cast<long long>(g) * per));
  const int e = min(vocab, b + per);
  const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;      // per is a multiple of 4, so b is one too

  float m = -INFINITY;
  {
    int i = b;
    if (vec)
      for (; i + 4 <= e; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(row + i);
        m = fmaxf(fmaxf(m, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
      }
    for (; i < e; ++i) m = fmaxf(m, row[i]);
  }
  m = block_max(m, red);
  if (threadIdx.x == 0) {
    block_m = m;
    winner = 0;
  }
  cluster.sync();
  for (int c = 0; c < nblocks; ++c) m = fmaxf(m, *cluster.map_shared_rank(&block_m, c));

  double s = 0.0;
  {
    int i = b;
    if (vec)
      for (; i + 4 <= e; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(row + i);
        s += static_cast<double>(expf((v.x - m) * inv_t));
        s += static_cast<double>(expf((v.y - m) * inv_t));
        s += static_cast<double>(expf((v.z - m) * inv_t));
        s += static_cast<double>(expf((v.w - m) * inv_t));
      }
    for (; i < e; ++i) s += static_cast<double>(expf((row[i] - m) * inv_t));
  }
  // running totals in id order: over the warp, over the block's warps, over the cluster's blocks
  double incl = s;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const double v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) warp_before[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const double w = warp_before[lane];
    double wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double v = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += v;
    }
    warp_before[lane] = wi - w;
    if (lane == 31) block_total = wi;
  }
  __syncthreads();
  const double before_in_block = warp_before[warp] + (incl - s);
  cluster.sync();
  double before = 0.0, total = 0.0;
  for (int c = 0; c < nblocks; ++c) {
    const double t = *cluster.map_shared_rank(&block_total, c);
    if (c < rank) before += t;
    total += t;
  }
  const double target = uniform[r] * total;
  const double begin = before + before_in_block;
  if (g == 0 || (s > 0.0 && begin <= target)) atomicMax(cluster.map_shared_rank(&winner, 0), g);
  cluster.sync();
  if (g == *cluster.map_shared_rank(&winner, 0)) {
    double u = target - begin;
    int pick = -1;
    for (int i = b; i < e; ++i) {
      u -= static_cast<double>(expf((row[i] - m) * inv_t));
      if (u < 0.0) { pick = i; break; }
    }
    if (pick < 0) {
      pick = vocab - 1;
      for (int i = e; i < vocab; ++i) {
        if (expf((row[i] - m) * inv_t) > 0.0f) { pick = i; break; }
      }
    }
    out[r] = pick;
  }
  cluster.sync();        // nobody leaves while another block may still read its shared memory
}

// Token feedback for a step launched before the previous step's tokens have reached the host: row r of the new
// step takes the id that the previous step chose at place src[r] of its output (src[r] < 0: keep what the host wrote).
__global__ void feedback_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ chosen,
                                       const int* __restrict__ src, int n) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < n && src[r] >= 0) token_ids[r] = chosen[ck_row(src[r])];   // checked against the length of `chosen`
}

}  // namespace dl

DL_EXPORT int dl_feedback_tokens(int* token_ids, const int* chosen, const int* src, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  dl::feedback_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(token_ids, chosen, src, n);
  return dl::launch_status();
}

// scratch: room for rows * 32 floats and rows * 32 ints (rows * 256 bytes), or null to use one block per row.
// status_dst (may be null): receives *status_src, so that a word some earlier kernel of the step may have written
// travels to the host in the same copy as the chosen ids.
DL_EXPORT int dl_argmax(const float* logits, int ld, int rows, int vocab, int* out, void* scratch,
                        const int* status_src, int* status_dst, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return DL_ERR_UNSUPPORTED;
  if (scratch != nullptr && vocab >= 8192 && rows <= 65535) {
    float* pv = static_cast<float*>(scratch);
    int* pi = reinterpret_cast<int*>(pv + static_cast<size_t>(rows) * dl::ARGMAX_PARTS);
    dim3 grid(dl::ARGMAX_PARTS, rows);
    dl::argmax_part_kernel<<<grid, 256, 0, stream>>>(logits, ld, vocab, pv, pi);
    dl::argmax_final_kernel<<<rows, 32, 0, stream>>>(pv, pi, out, status_src, status_dst);
    return dl::launch_status();
  }
  dl::argmax_kernel<<<rows, dl::SAMPLE_THREADS, 0, stream>>>(logits, ld, vocab, out, status_src, status_dst);
  return dl::launch_status();
}

// out[r] = the index among `parts` partial results (largest value, lowest index among equals) of row r, as a matrix
// product with the argmax epilogue leaves them: pv float [rows][parts], pi int [rows][parts].
DL_EXPORT int dl_argmax_of_parts(const float* pv, const int* pi, int rows, int parts, int* out, const int* status_src,
                                 int* status_dst, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (parts <= 0) return DL_ERR_UNSUPPORTED;
  return dl::launch_streaming(dl::argmax_of_parts_kernel, dim3(rows), dim3(256), 0, stream, pv, pi, parts, out,
                              status_src, status_dst);
}

// temperature: fp32 [rows] (> 0); uniform: double [rows] in [0, 1).
DL_EXPORT int dl_sample_temperature(const float* logits, int ld, int rows, int vocab, const float* temperature,
                                    const double* uniform, int* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return DL_ERR_UNSUPPORTED;
  // blocks per row: enough for runs of at most 16 ids a thread, a power of two, at most 8 (a portable cluster)
  int nblocks = 1;
  while (nblocks < 8 && static_cast<long long>(nblocks) * dl::SAMPLE_THREADS * 16 < vocab) nblocks *= 2;
  if (static_cast<long long>(rows) * nblocks > 0x7fffffffll) return DL_ERR_UNSUPPORTED;
  const long long threads = static_cast<long long>(nblocks) * dl::SAMPLE_THREADS;
  const int per = static_cast<int>(((vocab + threads - 1) / threads + 3) & ~3ll);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(rows * nblocks));
  cfg.blockDim = dim3(dl::SAMPLE_THREADS);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(nblocks);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, dl::sample_temperature_kernel, logits, ld, vocab, per, temperature,
                                             uniform, out));
}
