// Token selection on the device over fp32 logits rows: greedy argmax, temperature and min-p sampling by a walk down
// the ids, the penalties, and top-k / top-p sampling (further down, with their own account).
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
                          const double* __restrict__ cut_offset, int* __restrict__ out) {
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
  // min-p (cut_offset[r] = temperature * log(min_p), -inf or no array: off): logits below max + offset have no mass
  const double cut = cut_offset != nullptr ? static_cast<double>(m) + cut_offset[r] : -INFINITY;
  auto mass = [&](float l) {
    return static_cast<double>(l) >= cut ? static_cast<double>(expf((l - m) * inv_t)) : 0.0;
  };

  double s = 0.0;
  {
    int i = b;
    if (vec)
      for (; i + 4 <= e; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(row + i);
        s += mass(v.x);
        s += mass(v.y);
        s += mass(v.z);
        s += mass(v.w);
      }
    for (; i < e; ++i) s += mass(row[i]);
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
      u -= mass(row[i]);
      if (u < 0.0) { pick = i; break; }
    }
    if (pick < 0) {
      pick = vocab - 1;
      for (int i = e; i < vocab; ++i) {
        if (mass(row[i]) > 0.0) { pick = i; break; }
      }
    }
    out[r] = pick;
  }
  cluster.sync();        // nobody leaves while another block may still read its shared memory
}

// ---- penalties and the filtered draw (top-k, min-p, top-p) -----------------------------------------------------
//
// The reference's pipeline, penalties -> top-k -> temperature -> min-p -> top-p -> draw
// (dynalm/src/sampling/sampler.cpp:96-220), works on the candidates in the order (logit descending, id ascending).
// Here one block per row narrows the vocabulary down to the places in that order on which the pipeline turns (see
// sample_filtered_kernel); a row that does not fit gives -1 and is done by the host from its logits.

// Repetition, frequency and presence penalties (sampler.cpp:96-116): triple j = (selection, token id, count of the
// id in the request's recent context), ids unique within a selection and the triples of a selection next to one
// another (first[sel] .. first[sel + 1]); params[selection] = (repetition, frequency, presence). float32 arithmetic
// in the order of the host's, no fused multiply-add.
//
// A request that is decoded a step ahead has one token the host has not seen yet: the one the step in flight chose,
// chosen[pending[sel]] (pending[sel] < 0: none). It counts as the newest token of the context (the host leaves room
// for it in the window): a triple with its id counts one more, and if no triple has it, it is penalised as an id
// seen once (thread n_triples + sel looks for it among the selection's triples).
__device__ __forceinline__ void penalise(float* at, float rep, float freq, float pres, int count) {
  float l = *at;
  if (rep != 1.0f) l = l > 0.0f ? __fdiv_rn(l, rep) : __fmul_rn(l, rep);
  *at = __fsub_rn(l, __fadd_rn(__fmul_rn(static_cast<float>(count), freq), pres));
}

__global__ void apply_penalties_kernel(float* __restrict__ logits, int ld, int vocab, const int* __restrict__ rows,
                                       const int* __restrict__ triples, int n_triples, const float* __restrict__ params,
                                       const int* __restrict__ first, int n_sel, const int* __restrict__ chosen,
                                       const int* __restrict__ pending) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n_triples + (pending != nullptr ? n_sel : 0)) return;
  if (j < n_triples) {
    const int sel = triples[3 * j], id = triples[3 * j + 1];
    int count = triples[3 * j + 2];
    if (id < 0 || id >= vocab) return;
    if (pending != nullptr && pending[sel] >= 0 && chosen[pending[sel]] == id) ++count;
    penalise(logits + static_cast<size_t>(ck_row(rows[sel])) * ld + id, params[3 * sel], params[3 * sel + 1],
             params[3 * sel + 2], count);
    return;
  }
  const int sel = j - n_triples;
  if (pending[sel] < 0) return;
  const int id = chosen[pending[sel]];
  if (id < 0 || id >= vocab) return;
  for (int k = first[sel]; k < first[sel + 1]; ++k)
    if (triples[3 * k + 1] == id) return;                // counted there
  penalise(logits + static_cast<size_t>(ck_row(rows[sel])) * ld + id, params[3 * sel], params[3 * sel + 1],
           params[3 * sel + 2], 1);
}

constexpr int SAMPLE_CAP = 1024;          // candidates a row may keep (= threads of its block)
constexpr int SAMPLE_BINS = 2048;
constexpr double SAMPLE_FIXED = 1099511627776.0;      // 2^40: masses as integers, so that their sums have no order

// Inclusive running sum over the block's threads in thread order. `red`: 33 doubles.
__device__ __forceinline__ double block_scan_f64(double v, double* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const double x = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += x;
  }
  __syncthreads();
  if (lane == 31) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const double w = red[lane];
    double wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double x = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += x;
    }
    red[lane] = wi - w;
  }
  __syncthreads();
  return v + red[warp];
}

__device__ __forceinline__ int block_count(bool flag, int* red_i) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = __popc(__ballot_sync(0xffffffffu, flag));
  __syncthreads();
  if (lane == 0) red_i[warp] = c;
  __syncthreads();
  int t = 0;
  for (int w = 0; w < 32; ++w) t += red_i[w];
  __syncthreads();
  return t;
}

// Where a logit falls among SAMPLE_BINS equal steps from `lo` up (non-decreasing in l, whatever the rounding).
__device__ __forceinline__ int sample_bin(float l, float lo, float scale) {
  const float x = (l - lo) * scale;
  return x <= 0.0f ? 0 : (x >= static_cast<float>(SAMPLE_BINS - 1) ? SAMPLE_BINS - 1 : static_cast<int>(x));
}

// Inclusive running sum of integers over the block's threads in thread order. `red`: 33 words.
__device__ __forceinline__ unsigned long long block_scan_u64(unsigned long long v, unsigned long long* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long x = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += x;
  }
  __syncthreads();
  if (lane == 31) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const unsigned long long w = red[lane];
    unsigned long long wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long x = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += x;
    }
    red[lane] = wi - w;
    if (lane == 31) red[32] = wi;
  }
  __syncthreads();
  return v + red[warp];
}

// f(id, logit) for every id of the row, each thread of the block taking every SAMPLE_CAP-th group of four: sixteen
// logits are asked for before the first is used (a loop of single loads waits a trip to L2 per logit: 20 us a pass
// over 128,256 logits instead of 3). In no particular order: what the callers add up has none.
template <typename F>
__device__ __forceinline__ void sample_for_each(const float* __restrict__ row, int vocab, F f) {
  const int t = threadIdx.x;
  int done = 0;
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const int n4 = vocab >> 2;
    const float4* r4 = reinterpret_cast<const float4*>(row);
    int i = t;
    for (; i + 3 * SAMPLE_CAP < n4; i += 4 * SAMPLE_CAP) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = r4[i + u * SAMPLE_CAP];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int b = (i + u * SAMPLE_CAP) * 4;
        f(b, v[u].x); f(b + 1, v[u].y); f(b + 2, v[u].z); f(b + 3, v[u].w);
      }
    }
    for (; i < n4; i += SAMPLE_CAP) {
      const float4 v = r4[i];
      f(4 * i, v.x); f(4 * i + 1, v.y); f(4 * i + 2, v.z); f(4 * i + 3, v.w);
    }
    done = n4 << 2;
  }
  for (int i = done + t; i < vocab; i += SAMPLE_CAP) f(i, row[i]);
}

// The bins that narrow a row down, level by level: level n + 1 divides the chosen bin of level n again.
struct SampleBins {
  float lo[3], scale[3];
  int bin[3];
  int depth;
  // +1 above the chosen bins, 0 inside them, -1 below
  __device__ __forceinline__ int side(float l) const {
#pragma unroll
    for (int level = 0; level < 3; ++level) {
      if (level < depth) {
        const int b = sample_bin(l, lo[level], scale[level]);
        if (b != bin[level]) return b > bin[level] ? 1 : -1;
      }
    }
    return 0;
  }
};

// dparams[sel] = (temperature, temperature * log(min_p) or -inf, top_p, uniform); top_k[sel]: 0 = off.
//
// Both filters come down to finding a place in the order (logit descending, id ascending) by a running total from
// the top: of ids for top-k, of mass for top-p and for the draw. The row is narrowed to that place by histograms
// over equal steps of the logit, up to three levels deep, until the bin that holds the place has at most SAMPLE_CAP
// ids; those are sorted and the place is found among them. Masses are integers (expf(...) * 2^40, cut off), so that
// their sums do not depend on the order in which threads add them and a running total is exact.
//   top-k (with or without top-p): the ids at or above the bin of the k-th are the candidates (at most SAMPLE_CAP,
//     else the host); on them, sorted, the reference's pipeline in double precision.
//   top-p alone: the nucleus may be most of the vocabulary, so nothing but the bin of its last id is gathered:
//     the place where the running mass reaches top_p of the whole gives the mass kept, the place where it exceeds
//     uniform * kept gives the id.
__global__ void __launch_bounds__(SAMPLE_CAP)
sample_filtered_kernel(const float* __restrict__ logits, int ld, int vocab, const int* __restrict__ rows,
                       const double* __restrict__ dparams, const int* __restrict__ top_k, int* __restrict__ out) {
  // mass (or count) per bin, in two 32-bit halves: a 32-bit atomic add in shared memory is one instruction, and its
  // old value tells whether it carried
  __shared__ unsigned int hist_lo[SAMPLE_BINS], hist_hi[SAMPLE_BINS];
  __shared__ unsigned long long cand[SAMPLE_CAP];
  __shared__ unsigned long long red_u[33];
  __shared__ double red[33];
  __shared__ float redf[33];
  __shared__ int red_i[32];
  __shared__ int n_cand, picked_bin;
  __shared__ unsigned long long picked_rest, picked_above, picked_inside, found_cum;
  __shared__ int found_id;
  __shared__ double kept_s;
  const int sel = blockIdx.x, t = threadIdx.x;
  const int out_at = ck_row(rows[sel]);
  const float* row = logits + static_cast<size_t>(out_at) * ld;
  const double temp = dparams[4 * sel], cut_off = dparams[4 * sel + 1], top_p = dparams[4 * sel + 2];
  const double u = dparams[4 * sel + 3];
  const int k = top_k[sel];
  const bool use_k = k > 0 && k < vocab, use_p = top_p < 1.0;
  const float inv_t = static_cast<float>(1.0 / temp);
  if (!use_k && !use_p) {
    // neither filter is in effect: the reference then walks the ids in their own order, not in that of their
    // logits, which is the other kernel's walk; asked of this one, the row goes to the host
    if (t == 0) out[out_at] = -1;
    return;
  }

  // the largest and the smallest finite logit (NaN and -inf take no part anywhere below)
  float hi = -INFINITY, lo = INFINITY;
  sample_for_each(row, vocab, [&](int, float l) {
    if (l > -INFINITY) { hi = fmaxf(hi, l); lo = fminf(lo, l); }
  });
  const float mine_hi = hi;        // the largest logit this thread has seen: the threads' largest bound the place from below
  hi = block_max(hi, redf);
  lo = -block_max(-lo, redf);
  if (!(hi > -INFINITY) || !(hi < INFINITY)) {
    // nothing finite to choose from, or an infinite logit: no distribution to draw from; the row says so
    if (t == 0) out[out_at] = -1;
    return;
  }
  const double cut = static_cast<double>(hi) + cut_off;      // min-p: logits below it are out (sampler.cpp:146)
  // (in float32 alone: the smallest float at or above the cut stands for it, and the product with 2^40 is exact)
  float cut_f = static_cast<float>(cut);
  if (static_cast<double>(cut_f) < cut) cut_f = nextafterf(cut_f, INFINITY);
  auto mass = [&](float l) -> unsigned long long {
    return l >= cut_f ? __float2ull_rz(expf((l - hi) * inv_t) * static_cast<float>(SAMPLE_FIXED)) : 0ull;
  };
  auto sort_key = [](float l, unsigned int id) {            // ascending in this key = (logit descending, id ascending)
    const unsigned int bits = __float_as_uint(l);
    const unsigned int rising = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);     // grows with the logit
    return (static_cast<unsigned long long>(~rising) << 32) | id;
  };
  auto key_logit = [](unsigned long long key) {
    const unsigned int rising = ~static_cast<unsigned int>(key >> 32);
    return __uint_as_float((rising & 0x80000000u) ? (rising & 0x7fffffffu) : ~rising);
  };
  auto sort_cand = [&]() {                                  // all SAMPLE_CAP places of cand, ascending
    for (int size = 2; size <= SAMPLE_CAP; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        const int other = t ^ stride;
        if (other > t) {
          const unsigned long long a = cand[t], b = cand[other];
          const bool up = (t & size) == 0;
          if ((a > b) == up) { cand[t] = b; cand[other] = a; }
        }
        __syncthreads();
      }
    }
  };
  // A floor under the place that is looked for, from the threads' largest logits alone (every one of them is a logit
  // of the row, so at least j ids lie at or above the j-th largest of them, with at least their mass): ids below the
  // floor need not be counted or weighed, which leaves the histograms a few thousand ids instead of the vocabulary.
  // `reach`: how many ids (by_count) or how much mass the place needs from the top.
  auto floor_from_thread_maxima = [&](unsigned long long reach, bool by_count) -> float {
    __syncthreads();
    cand[t] = mine_hi > -INFINITY ? sort_key(mine_hi, static_cast<unsigned int>(t)) : ~0ull;
    __syncthreads();
    sort_cand();
    const bool real = cand[t] != ~0ull;
    const float mine = real ? key_logit(cand[t]) : 0.0f;
    const unsigned long long w = !real ? 0ull : (by_count ? 1ull : mass(mine));
    const unsigned long long incl = block_scan_u64(w, red_u);
    if (t == 0) found_id = -1;
    __syncthreads();
    if (incl - w < reach && incl >= reach) found_id = t;     // the first thread maximum at which the running total reaches it
    __syncthreads();
    const int at = found_id;
    const float floor = at >= 0 ? key_logit(cand[at]) : -INFINITY;
    __syncthreads();
    return floor;
  };
  float floor = -INFINITY;
  auto counted = [&](float l) { return l > -INFINITY && l >= floor; };

  SampleBins bins;
  // One or more levels of narrowing: the row (at level 0) or the bin chosen at the level before is divided into
  // SAMPLE_BINS equal steps, and the bin is chosen in which the running total from the top (of ids if by_count, else
  // of mass) reaches `rest` >= 1. Returns what of `rest` is left to find inside that bin. By count, *ids_above grows
  // by the ids in the bins above it and *ids_inside becomes the ids in it (by mass nobody counts: one atomic less
  // per id). If even the lowest bin does not reach it, that bin is chosen.
  auto narrow = [&](unsigned long long rest, bool by_count, int first_level, int last_level, int* ids_above,
                    int* ids_inside) -> unsigned long long {
#pragma unroll
    for (int level = 0; level < 3; ++level) {
      if (level < first_level || level > last_level) continue;
      bins.depth = level;
      bins.lo[level] = level == 0 ? lo : bins.lo[level - 1] + static_cast<float>(bins.bin[level - 1]) / bins.scale[level - 1];
      bins.scale[level] = level == 0 ? (hi > lo ? static_cast<float>(SAMPLE_BINS) / (hi - lo) : 0.0f)
                                     : bins.scale[level - 1] * static_cast<float>(SAMPLE_BINS);
      if (level > 0 && !(bins.scale[level - 1] > 0.0f)) { bins.lo[level] = lo; bins.scale[level] = 0.0f; }
      for (int b = t; b < SAMPLE_BINS; b += SAMPLE_CAP) { hist_lo[b] = 0; hist_hi[b] = 0; }
      __syncthreads();
      sample_for_each(row, vocab, [&](int, float l) {
        if (!counted(l) || bins.side(l) != 0) return;
        const unsigned long long w = by_count ? 1ull : mass(l);
        if (w == 0) return;
        const int b = sample_bin(l, bins.lo[level], bins.scale[level]);
        const unsigned int low = static_cast<unsigned int>(w), high = static_cast<unsigned int>(w >> 32);
        const unsigned int old = atomicAdd(&hist_lo[b], low);
        const unsigned int carry = old + low < old ? 1u : 0u;
        if (high + carry != 0) atomicAdd(&hist_hi[b], high + carry);
      });
      __syncthreads();
      auto hist = [&](int b) { return (static_cast<unsigned long long>(hist_hi[b]) << 32) | hist_lo[b]; };
      // thread t owns bins SAMPLE_BINS-1-2t and SAMPLE_BINS-2-2t: a running sum over threads runs from the top bin down
      const int b_hi = SAMPLE_BINS - 1 - 2 * t, b_lo = b_hi - 1;
      const unsigned long long h_hi = hist(b_hi), h_lo = hist(b_lo);
      const unsigned long long incl = block_scan_u64(h_hi + h_lo, red_u);
      const unsigned long long all = red_u[32];
      const unsigned long long before = incl - (h_hi + h_lo);
      if (t == 0) {      // out of reach (more than the whole): the lowest bin, everything else above it
        picked_bin = 0;
        picked_rest = rest;
        picked_above = all - hist(0);
        picked_inside = hist(0);
      }
      __syncthreads();
      if (before < rest && incl >= rest) {          // exactly one thread (none if out of reach)
        if (before + h_hi >= rest) {
          picked_bin = b_hi; picked_rest = rest - before; picked_above = before; picked_inside = h_hi;
        } else {
          picked_bin = b_lo; picked_rest = rest - before - h_hi; picked_above = before + h_hi; picked_inside = h_lo;
        }
      }
      __syncthreads();
      bins.bin[level] = picked_bin;
      bins.depth = level + 1;
      rest = picked_rest;
      if (by_count) {
        *ids_above += static_cast<int>(picked_above);
        *ids_inside = static_cast<int>(picked_inside);
      }
      __syncthreads();
    }
    return rest;
  };
  // Thread t's own stretch of ids, for what has to go by the order of the ids.
  const int per = (vocab + SAMPLE_CAP - 1) / SAMPLE_CAP;
  const int own_b = min(vocab, t * per), own_e = min(vocab, own_b + per);
  // Whether the ids inside the chosen bins all have one logit (after three levels a bin is narrower than the
  // step between two floats, unless the row's range is absurd); *value = that logit.
  auto one_value = [&](float* value) -> bool {
    float most = -INFINITY, least = INFINITY;
    sample_for_each(row, vocab, [&](int, float l) {
      if (counted(l) && bins.side(l) == 0) { most = fmaxf(most, l); least = fminf(least, l); }
    });
    most = block_max(most, redf);
    least = -block_max(-least, redf);
    *value = most;
    return most == least;
  };
  // The id of the j-th (from 0) of the ids inside the chosen bins, in the order of the ids; -1 if there are fewer.
  auto nth_inside = [&](unsigned long long j) -> int {
    unsigned long long mine = 0;
    for (int i = own_b; i < own_e; ++i) mine += counted(row[i]) && bins.side(row[i]) == 0;
    const unsigned long long incl = block_scan_u64(mine, red_u);
    if (t == 0) found_id = -1;
    __syncthreads();
    if (incl - mine <= j && j < incl) {
      unsigned long long seen = incl - mine;
      for (int i = own_b; i < own_e; ++i) {
        if (counted(row[i]) && bins.side(row[i]) == 0 && seen++ == j) { found_id = i; break; }
      }
    }
    __syncthreads();
    return found_id;
  };
  // The ids inside the chosen bins (and above them, if `with_above`) into cand, sorted by (logit descending, id
  // ascending); the number of them, or -1 if they are more than cand holds. inside_limit >= 0: of those inside only the first
  // inside_limit in the order of the ids (they have one logit, so these come first in the order of the candidates).
  auto gather_sorted = [&](bool with_above, long long inside_limit) -> int {
    if (t == 0) n_cand = 0;
    __syncthreads();
    auto put = [&](int i, float l) {
      const int at = atomicAdd(&n_cand, 1);
      if (at < SAMPLE_CAP) cand[at] = sort_key(l, static_cast<unsigned int>(i));
    };
    sample_for_each(row, vocab, [&](int i, float l) {
      if (!counted(l)) return;
      const int side = bins.side(l);
      if (side < 0 || (side > 0 && !with_above) || (side == 0 && inside_limit >= 0)) return;
      put(i, l);
    });
    if (inside_limit >= 0) {
      unsigned long long mine = 0;
      for (int i = own_b; i < own_e; ++i) mine += counted(row[i]) && bins.side(row[i]) == 0;
      unsigned long long rank = block_scan_u64(mine, red_u) - mine;
      for (int i = own_b; i < own_e; ++i) {
        const float l = row[i];
        if (counted(l) && bins.side(l) == 0 && rank++ < static_cast<unsigned long long>(inside_limit)) put(i, l);
      }
    }
    __syncthreads();
    const int n = n_cand;
    __syncthreads();
    if (n > SAMPLE_CAP) return -1;
    if (n == 0) return 0;
    if (t >= n) cand[t] = ~0ull;
    __syncthreads();
    sort_cand();
    return n;
  };

  if (!use_k) {
    // ---- top-p alone ----
    unsigned long long mine = 0;
    sample_for_each(row, vocab, [&](int, float l) { mine += mass(l); });
    block_scan_u64(mine, red_u);
    const unsigned long long total = red_u[32];
    __syncthreads();
    // The first place (in the order) where the running mass reaches x: its id, and the running mass there.
    auto locate = [&](unsigned long long x) -> bool {
      unsigned long long rest = narrow(x, false, 0, 1, nullptr, nullptr);
      int n = gather_sorted(false, -1);
      if (n < 0) {                                       // the bin of two levels holds too many: a third
        rest = narrow(rest, false, 2, 2, nullptr, nullptr);
        n = gather_sorted(false, -1);
      }
      if (n < 0) {
        // more ids at the place than can be sorted: they have one logit, so one mass, and their order is that of
        // the ids
        float value;
        if (!one_value(&value)) return false;
        const unsigned long long w = mass(value);
        if (w == 0) return false;
        const unsigned long long j = (rest + w - 1) / w - 1;
        const int id = nth_inside(j);
        if (id < 0) return false;
        if (t == 0) found_cum = (x - rest) + (j + 1) * w;
        __syncthreads();
        return true;
      }
      if (n == 0) return false;
      const int id = static_cast<int>(cand[t] & 0xffffffffull);
      const unsigned long long w = t < n ? mass(row[id]) : 0ull;
      const unsigned long long cum = block_scan_u64(w, red_u);
      const int pos = block_count(t < n && cum < rest, red_i);
      if (pos >= n) return false;                      // the bin does not hold the place after all
      if (t == pos) { found_id = id; found_cum = (x - rest) + cum; }
      __syncthreads();
      return true;
    };
    if (total == 0) {
      if (t == 0) out[out_at] = -1;
      return;
    }
    unsigned long long share = static_cast<unsigned long long>(top_p * static_cast<double>(total));
    share = share < 1 ? 1 : (share > total ? total : share);
    floor = floor_from_thread_maxima(share, false);          // the draw's place lies at or above the nucleus' end
    if (floor > lo) lo = floor;
    if (!locate(share)) {
      if (t == 0) out[out_at] = -1;
      return;
    }
    const unsigned long long kept = found_cum;          // the mass of the nucleus (sampler.cpp:196-205)
    __syncthreads();
    unsigned long long aim = static_cast<unsigned long long>(u * static_cast<double>(kept));
    if (aim >= kept) aim = kept - 1;
    if (!locate(aim + 1)) {                             // the first place where the running mass exceeds u * kept
      if (t == 0) out[out_at] = -1;
      return;
    }
    if (t == 0) out[out_at] = found_id;
    return;
  }

  // ---- top-k, with or without top-p ----
  floor = floor_from_thread_maxima(static_cast<unsigned long long>(k), true);
  if (floor > lo) lo = floor;
  int ids_above = 0, ids_inside = 0;
  unsigned long long inside_wanted = static_cast<unsigned long long>(k);
  for (int level = 0; level < 3; ++level) {              // until the ids above and inside fit the candidates
    inside_wanted = narrow(inside_wanted, true, level, level, &ids_above, &ids_inside);
    if (ids_above + ids_inside <= SAMPLE_CAP) break;
  }
  long long inside_limit = -1;
  if (ids_above + ids_inside > SAMPLE_CAP && k <= SAMPLE_CAP) {
    // more ids with the k-th logit than can be kept: of those (one logit) the first in the order of the ids
    float value;
    if (one_value(&value)) inside_limit = static_cast<long long>(inside_wanted);
  }
  const int n = gather_sorted(true, inside_limit);
  if (n <= 0) {
    if (t == 0) out[out_at] = -1;
    return;
  }
  // the pipeline on the sorted candidates, thread i = candidate i
  const int id = static_cast<int>(cand[t] & 0xffffffffull);
  const double l = t < n ? static_cast<double>(row[id]) : 0.0;
  const int k_eff = min(k, n);
  const bool valid = t < k_eff && l >= cut;
  const int m = block_count(valid, red_i);             // sorted: the valid ones are the first m
  if (m == 0) {
    if (t == 0) out[out_at] = static_cast<int>(cand[0] & 0xffffffffull);        // cannot be: the largest logit passes
    return;
  }
  double prob = valid ? exp((l - static_cast<double>(hi)) / temp) : 0.0;
  double cum = block_scan_f64(prob, red);
  if (t == m - 1) kept_s = cum;
  __syncthreads();
  double kept = kept_s;
  int keep = m;
  if (use_p) {
    const double share = top_p * kept;                   // with top-k, top-p applies to what top-k kept
    keep = block_count(valid && cum < share, red_i) + 1;           // first place where the running mass reaches it
    keep = max(1, min(keep, m));
    __syncthreads();
    if (t == keep - 1) kept_s = cum;
    __syncthreads();
    kept = kept_s;
  }
  const double aim = u * kept;
  int pick = block_count(t < keep && cum <= aim, red_i);           // first place where the running mass exceeds it
  pick = min(pick, keep - 1);
  if (t == pick) out[out_at] = id;
}

// Token feedback for a step launched before the previous step's tokens have reached the host: row r of the new
// step takes the id that the previous step chose at place src[r] of its output (src[r] < 0: keep what the host wrote).
__global__ void feedback_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ chosen,
                                       const int* __restrict__ src, int n) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < n && src[r] >= 0) {
    const int id = chosen[ck_row(src[r])];   // checked against the length of `chosen`
    token_ids[r] = id < 0 ? 0 : id;          // a row the sampling kernel could not decide (-1): the host finds it when
                                             // it reads the ids and fails the request; the step in flight stays in bounds
  }
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

// rows: the logits rows of the n_sel selections; triples: int32 [n_triples][3] = (selection, token id, count), those
// of a selection next to one another, first: int32 [n_sel + 1] where each selection's begin; params: fp32 [n_sel][3] =
// (repetition, frequency, presence). chosen, pending (both or neither): pending[sel] >= 0 names the place in `chosen`
// of a token of that selection's context that only the device knows yet. In place.
DL_EXPORT int dl_apply_penalties(float* logits, int ld, int vocab, const int* rows, const int* triples, int n_triples,
                                 const float* params, const int* first, int n_sel, const int* chosen,
                                 const int* pending, cudaStream_t stream) {
  if (n_sel <= 0 || (n_triples <= 0 && pending == nullptr)) return 0;
  if (vocab <= 0 || n_triples < 0 || first == nullptr || (pending != nullptr && chosen == nullptr)) return DL_ERR_UNSUPPORTED;
  const int threads = n_triples + (pending != nullptr ? n_sel : 0);
  dl::apply_penalties_kernel<<<(threads + 127) / 128, 128, 0, stream>>>(logits, ld, vocab, rows, triples, n_triples, params,
                                                                        first, n_sel, chosen, pending);
  return dl::launch_status();
}

// One draw per selection through top-k, min-p and top-p. rows: int32 [n_sel], the logits row of each;
// dparams: double [n_sel][4] = (temperature, temperature * log(min_p) or -inf, top_p, uniform in [0, 1));
// top_k: int32 [n_sel], 0 = off. out[rows[sel]]: the id, or -1 where the row has to be done by the host.
DL_EXPORT int dl_sample_filtered(const float* logits, int ld, int vocab, const int* rows, int n_sel,
                                 const double* dparams, const int* top_k, int* out, cudaStream_t stream) {
  if (n_sel <= 0) return 0;
  if (vocab <= 0) return DL_ERR_UNSUPPORTED;
  dl::sample_filtered_kernel<<<n_sel, dl::SAMPLE_CAP, 0, stream>>>(logits, ld, vocab, rows, dparams, top_k, out);
  return dl::launch_status();
}

// temperature: fp32 [rows] (> 0); uniform: double [rows] in [0, 1).
// cut_offset (may be null): double [rows], temperature * log(min_p) per row, -inf where min-p is off.
DL_EXPORT int dl_sample_temperature(const float* logits, int ld, int rows, int vocab, const float* temperature,
                                    const double* uniform, const double* cut_offset, int* out, cudaStream_t stream) {
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
                                             uniform, cut_offset, out));
}
