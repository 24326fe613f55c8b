// Drift metric of the redundancy-profiling pass: how far a layer's output moved since the previous
// denoising step, as mean|cur - prev| / mean|prev| over the positions where neither value is NaN.
// One pass over both tensors, no host synchronisation: every block reduces a fixed tile and leaves
// four partial sums in scratch memory; the block that takes the last ticket folds the partials,
// forms the ratio and adds it to a device-resident accumulator.
//
// Scratch layout: [0, 4) ticket counter (zero on entry, left zero on exit), pad to 256 bytes, then
// blocks x 4 doubles {sum|cur-prev|, sum|prev|, sum|cur|, count}.
#include "drift_stats.cuh"

#include "../../include/ditango_b200.h"
#include "errors.cuh"

#include <mutex>

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

// ------------------------------------------------------------------------------------------------
// Variant for callers that must not allocate: the scratch lives in this library's own device image.
//
// Some hosts of this library cannot give it memory at call time: an inference server that hands its
// whole device budget to its own pool at start-up and forbids later cudaMalloc (which would also
// stall every stream of the process while it runs), or a plug-in interface that passes inputs and
// outputs only.  For them the per-block partial sums go into a fixed array that every process
// loading the library carries on each GPU it uses, from load until exit (1 MiB).
namespace {

constexpr int64_t kStaticBlocks = 32760;                                           // 1 MiB in all
constexpr int64_t kStaticBytes = dtb::kDriftScratchHeader + kStaticBlocks * 4 * 8;
static_assert(kStaticBytes == (1 << 20), "static drift scratch is meant to be exactly 1 MiB");

static __device__ __align__(256) unsigned char g_drift_static_scratch[kStaticBytes];

// In host code the array's name is only a handle for the runtime, not a device address: the address
// is looked up once per device, with that device current, and kept here.
unsigned char* g_static_ptr[64] = {};
std::mutex g_static_mu;

int static_scratch(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64)
    return dtb::set_error(DTB_ERR_CUDA, "dtb_drift_accumulate_noalloc: cudaGetDevice failed: %s", cudaGetErrorString(e));
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_drift_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return dtb::set_error(DTB_ERR_CUDA, "dtb_drift_accumulate_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_static_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_static_ptr[dev];
  return DTB_OK;
}

}  // namespace

extern "C" {

DTB_API int64_t dtb_drift_noalloc_max_elements(void) { return kStaticBlocks * dtb::kDriftTile; }

DTB_API int dtb_drift_accumulate_noalloc(const float* cur, const float* prev, int64_t n, float* accum, void* stream) {
  if (n < 0) return dtb::set_error(DTB_ERR_ARG, "dtb_drift_accumulate_noalloc: negative length");
  if (!accum || (n > 0 && (!cur || !prev))) return dtb::set_error(DTB_ERR_ARG, "dtb_drift_accumulate_noalloc: null pointer");
  if (dtb::drift_blocks(n) > kStaticBlocks)
    return dtb::set_error(DTB_ERR_ARG,
                          "dtb_drift_accumulate_noalloc: n = %lld exceeds the %lld elements the built-in scratch covers; "
                          "use dtb_drift_accumulate with caller-provided scratch",
                          static_cast<long long>(n), static_cast<long long>(kStaticBlocks * dtb::kDriftTile));
  int rc = dtb::require_sm100();
  if (rc != DTB_OK) return rc;
  unsigned char* scratch = nullptr;
  rc = static_scratch(&scratch);
  if (rc != DTB_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left.  Only the ticket counter has to start at zero
  // (a call that ran to completion leaves it so; this also covers one that did not).
  cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(unsigned int), s);
  if (e == cudaSuccess) e = dtb::launch_drift_stats(cur, prev, n, accum, scratch, s);
  if (e != cudaSuccess) return dtb::set_error(DTB_ERR_CUDA, "dtb_drift_accumulate_noalloc failed: %s", cudaGetErrorString(e));
  return DTB_OK;
}

}  // extern "C"
