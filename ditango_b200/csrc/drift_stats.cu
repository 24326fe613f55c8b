// Drift metric of the redundancy-profiling pass: how far a layer's output moved since the previous
// denoising step, as mean|cur - prev| / mean|prev| over the positions where neither value is NaN.
// One pass over both tensors, no host synchronisation: every block reduces a fixed tile and leaves
// four partial sums in scratch memory; the block that takes the last ticket folds the partials,
// forms the ratio and adds it to a device-resident accumulator.
//
// Scratch layout: [0, 4) ticket counter (zero on entry, left zero on exit), pad to 256 bytes, then
// blocks x 4 doubles {sum|cur-prev|, sum|prev|, sum|cur|, count}.
#include "drift_stats.cuh"

#include <math.h>

namespace dtb {

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sums of the calling block's four per-thread values; valid in thread 0.
__device__ __forceinline__ void block_sum4(double (&v)[4], double (*smem)[4]) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = warp_sum(v[i]);
  if (lane == 0)
    for (int i = 0; i < 4; ++i) smem[warp][i] = v[i];
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      double x = (lane < kThreads / 32) ? smem[lane][i] : 0.0;
      v[i] = warp_sum(x);
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void add_elem(float c, float p, float& d, float& o, float& n, float& k) {
  if (c == c && p == p) {      // neither is NaN
    d += fabsf(c - p);
    o += fabsf(p);
    n += fabsf(c);
    k += 1.f;
  }
}

}  // namespace

__global__ void __launch_bounds__(kThreads) drift_stats_kernel(const float* __restrict__ cur,
                                                               const float* __restrict__ prev, int64_t n,
                                                               float* accum, unsigned char* scratch) {
  __shared__ double red[kThreads / 32][4];
  __shared__ bool is_last;
  unsigned int* ticket = reinterpret_cast<unsigned int*>(scratch);
  double* partials = reinterpret_cast<double*>(scratch + kDriftScratchHeader);

  const int64_t tile0 = static_cast<int64_t>(blockIdx.x) * kDriftTile;
  const int64_t tile1 = (tile0 + kDriftTile < n) ? tile0 + kDriftTile : n;
  float d = 0.f, o = 0.f, m = 0.f, k = 0.f;   // <= 64 elements per thread: fp32 is exact enough here
  const bool aligned = ((reinterpret_cast<uintptr_t>(cur) | reinterpret_cast<uintptr_t>(prev)) & 15) == 0;
  if (aligned) {
    for (int64_t i = tile0 + threadIdx.x * 4; i < tile1; i += kThreads * 4) {
      if (i + 4 <= tile1) {
        const float4 c = __ldcs(reinterpret_cast<const float4*>(cur + i));
        const float4 p = __ldcs(reinterpret_cast<const float4*>(prev + i));
        add_elem(c.x, p.x, d, o, m, k);
        add_elem(c.y, p.y, d, o, m, k);
        add_elem(c.z, p.z, d, o, m, k);
        add_elem(c.w, p.w, d, o, m, k);
      } else {
        for (int64_t j = i; j < tile1; ++j) add_elem(cur[j], prev[j], d, o, m, k);
      }
    }
  } else {
    for (int64_t i = tile0 + threadIdx.x; i < tile1; i += kThreads) add_elem(cur[i], prev[i], d, o, m, k);
  }
  double v[4] = {d, o, m, k};
  block_sum4(v, red);
  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; ++i) partials[static_cast<int64_t>(blockIdx.x) * 4 + i] = v[i];
    __threadfence();
    is_last = (atomicAdd(ticket, 1u) == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;

  __threadfence();
  double t[4] = {0.0, 0.0, 0.0, 0.0};
  for (unsigned int b = threadIdx.x; b < gridDim.x; b += kThreads)
    for (int i = 0; i < 4; ++i) t[i] += __ldcg(&partials[static_cast<int64_t>(b) * 4 + i]);
  block_sum4(t, red);
  if (threadIdx.x == 0) {
    float rel;
    if (t[3] <= 0.0) {
      rel = INFINITY;                                   // no position without NaN
    } else {
      const double ori_mean = t[1] / t[3];
      const double val = (ori_mean < 1e-6) ? t[2] / t[3] : (t[0] / t[3]) / (ori_mean + 1e-8);
      rel = isfinite(val) ? static_cast<float>(val) : INFINITY;
    }
    *accum += rel;
    *ticket = 0u;                                       // ready for the next call on this scratch
  }
}

cudaError_t launch_drift_stats(const float* cur, const float* prev, int64_t n, float* accum, unsigned char* scratch,
                               cudaStream_t stream) {
  const int64_t blocks = drift_blocks(n);
  drift_stats_kernel<<<static_cast<unsigned int>(blocks), kThreads, 0, stream>>>(cur, prev, n, accum, scratch);
  return cudaGetLastError();
}

}  // namespace dtb
