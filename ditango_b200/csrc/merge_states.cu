// N-way merge of partial softmax-attention states in one pass over HBM.
//
// A "row" is one (token, head) pair: D values per state plus one log-sum-exp per state.  A group of
// D/4 lanes owns a row (4 fp32 or 4 bf16 values per lane, 128-bit / 64-bit accesses); lane i of the
// group fetches lse_i, the group reduces max and sum with shuffles, and every lane then pulls the
// weight of state i from lane i.
// Traffic per row: reads sum_i (D * sizeof(state i) + 4) bytes, writes 4*D + 4 (+ 2*D) bytes.
#include "merge_states.cuh"

#include <cuda_bf16.h>
#include <math.h>

namespace dtb {

namespace {

__device__ __forceinline__ float4 ld_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ float4 ld_bf4(const uint16_t* p) {
  uint32_t a, b;
  asm volatile("ld.global.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(a), "=r"(b) : "l"(p));
  float4 v;
  v.x = __uint_as_float(a << 16);
  v.y = __uint_as_float(a & 0xffff0000u);
  v.z = __uint_as_float(b << 16);
  v.w = __uint_as_float(b & 0xffff0000u);
  return v;
}
__device__ __forceinline__ void st_f4(float* p, float4 v) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void st_bf4(uint16_t* p, float4 v) {
  uint32_t a, b;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(a) : "f"(v.y), "f"(v.x));
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(b) : "f"(v.w), "f"(v.z));
  asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}

// Offset of row = (b*S + s)*H + h in an lse tensor.  Rows fit 32 bits (checked by the launcher), so
// the two divisions are 32-bit.
__device__ __forceinline__ uint32_t lse_offset(int layout, uint32_t row, uint32_t H, uint32_t S) {
  if (layout == 1) return row;                    // [B,S,H]
  const uint32_t tok = row / H;
  const uint32_t h = row - tok * H;
  const uint32_t b = tok / S;
  const uint32_t s = tok - b * S;
  return (b * H + h) * S + s;                     // [B,H,S]
}

}  // namespace

// G = lanes per row = D/4.  U rows per group in flight, states fetched CH at a time: every thread
// keeps CH*U 16-byte loads outstanding and issues them before it touches the weights, so the lse
// round trip and the value round trips overlap instead of queueing behind one another.
template <int G, int U, int CH>
__global__ void __launch_bounds__(128) merge_states_kernel(const MergeParams p) {
  constexpr int D = G * 4;
  constexpr int kGroupsPerWarp = 32 / G;
  const int lane_in_group = threadIdx.x % G;
  const int64_t warp_id = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / 32;
  const int64_t n_warps = static_cast<int64_t>(gridDim.x) * blockDim.x / 32;
  const int group_in_warp = (threadIdx.x % 32) / G;
  const unsigned full = 0xffffffffu;
  const int n = p.nstates;

  auto load_chunk = [&](int c0, int64_t base, float4 (&v)[CH][U]) {
#pragma unroll
    for (int k = 0; k < CH; ++k) {
      if (c0 + k < n) {
        const bool f32 = p.out_dtype[c0 + k] == 0;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int64_t row = base + u;
          if (row < p.rows) {
            const int64_t off = row * D + lane_in_group * 4;
            v[k][u] = f32 ? ld_f4(static_cast<const float*>(p.outs[c0 + k]) + off)
                          : ld_bf4(static_cast<const uint16_t*>(p.outs[c0 + k]) + off);
          } else {
            v[k][u] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
      }
    }
  };

  // The loop bound is the same for every lane of a warp (shuffles below use the full mask); rows
  // past the end are guarded individually.
  for (int64_t wbase = warp_id * kGroupsPerWarp * U; wbase < p.rows; wbase += n_warps * kGroupsPerWarp * U) {
    const int64_t base = wbase + group_in_warp * U;
    float my[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t row = base + u;
      my[u] = -INFINITY;
      if (row < p.rows && lane_in_group < n)
        my[u] = p.lse[lane_in_group][lse_offset(p.lse_layout[lane_in_group], static_cast<uint32_t>(row), p.H, p.S)];
    }
    float4 v[CH][U];
    load_chunk(0, base, v);

    float w[U];        // this lane's weight (state index = lane_in_group)
    float lse_out[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float mx = my[u];
#pragma unroll
      for (int o = G / 2; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(full, mx, o, G));
      const float e = (my[u] == -INFINITY) ? 0.f : __expf(my[u] - mx);
      float sum = e;
#pragma unroll
      for (int o = G / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(full, sum, o, G);
      w[u] = (sum > 0.f) ? e / sum : 0.f;
      lse_out[u] = (sum > 0.f) ? mx + __logf(sum) : -INFINITY;
    }
    float4 acc[U];
#pragma unroll
    for (int u = 0; u < U; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c0 = 0; c0 < n; c0 += CH) {
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        if (c0 + k < n) {
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const float wi = __shfl_sync(full, w[u], c0 + k, G);
            // a state with weight 0 may hold anything (even inf/nan): it must not reach the sum
            if (wi != 0.f) {
              acc[u].x = fmaf(wi, v[k][u].x, acc[u].x);
              acc[u].y = fmaf(wi, v[k][u].y, acc[u].y);
              acc[u].z = fmaf(wi, v[k][u].z, acc[u].z);
              acc[u].w = fmaf(wi, v[k][u].w, acc[u].w);
            }
          }
        }
      }
      if (c0 + CH < n) load_chunk(c0 + CH, base, v);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t row = base + u;
      if (row < p.rows) {
        const int64_t off = row * D + lane_in_group * 4;
        if (p.out != nullptr) st_f4(p.out + off, acc[u]);
        if (p.out_bf16 != nullptr) st_bf4(p.out_bf16 + off, acc[u]);
        if (p.lse_out != nullptr && lane_in_group == 0)
          p.lse_out[lse_offset(p.lse_out_layout, static_cast<uint32_t>(row), p.H, p.S)] = lse_out[u];
      }
    }
  }
}

template <int U, int CH>
static cudaError_t launch_merge_cfg(const MergeParams& p, int G, int sm_count, cudaStream_t stream) {
  constexpr int kThreads = 128;
  const int64_t groups_needed = (p.rows + U - 1) / U;
  const int64_t blocks_needed = (groups_needed * G + kThreads - 1) / kThreads + 1;
  // one resident wave: CTAs per SM as the occupancy calculator reports them for this instantiation
  int per_sm = 0;
  cudaError_t oe = (G == 16)
      ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, merge_states_kernel<16, U, CH>, kThreads, 0)
      : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, merge_states_kernel<32, U, CH>, kThreads, 0);
  if (oe != cudaSuccess || per_sm < 1) per_sm = 6;
  const int64_t cap = static_cast<int64_t>(sm_count) * per_sm;
  int blocks = static_cast<int>(blocks_needed < cap ? blocks_needed : cap);
  if (blocks < 1) blocks = 1;
  if (G == 16)
    merge_states_kernel<16, U, CH><<<blocks, kThreads, 0, stream>>>(p);
  else
    merge_states_kernel<32, U, CH><<<blocks, kThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

// Rows per thread x states per fetch are chosen so that about eight 16-byte loads are outstanding
// per thread whatever the number of states: 4 rows x 2 states, 3 x 3, or 2 x 4.
cudaError_t launch_merge(const MergeParams& p, int head_dim, int sm_count, cudaStream_t stream) {
  const int G = head_dim / 4;
  if (p.rows >= (1ll << 31)) return cudaErrorInvalidValue;
#ifndef DTB_MERGE_FIXED_CFG
  if (p.nstates <= 2) return launch_merge_cfg<4, 2>(p, G, sm_count, stream);
  if (p.nstates == 3) return launch_merge_cfg<3, 3>(p, G, sm_count, stream);
#endif
  return launch_merge_cfg<2, 4>(p, G, sm_count, stream);
}

// ------------------------------------------------------------------------------------------------
// Strided chunk copy (head <-> sequence re-layouts around the Ulysses all-to-all).
// One CTA row of threads walks the 16-byte vectors of a chunk; grid-stride over chunks.
__global__ void __launch_bounds__(256) copy_chunks_kernel(const CopyParams p) {
  const int pair = blockIdx.y;
  const uint8_t* src = static_cast<const uint8_t*>(p.src[pair]);
  uint8_t* dst = static_cast<uint8_t*>(p.dst[pair]);
  const int64_t vec_per_chunk = p.chunk_bytes >> 4;
  const int64_t total = p.n0 * p.n1 * p.n2 * vec_per_chunk;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t chunk = i / vec_per_chunk;
    const int64_t v = i - chunk * vec_per_chunk;
    const int64_t i2 = chunk % p.n2;
    const int64_t t = chunk / p.n2;
    const int64_t i1 = t % p.n1;
    const int64_t i0 = t / p.n1;
    const uint4 val = __ldcs(reinterpret_cast<const uint4*>(src + i0 * p.ss0 + i1 * p.ss1 + i2 * p.ss2) + v);
    __stcs(reinterpret_cast<uint4*>(dst + i0 * p.ds0 + i1 * p.ds1 + i2 * p.ds2) + v, val);
  }
}

cudaError_t launch_copy_chunks(const CopyParams& p, int npairs, int sm_count, cudaStream_t stream) {
  const int64_t total = p.n0 * p.n1 * p.n2 * (p.chunk_bytes >> 4);
  int64_t blocks_needed = (total + 255) / 256;
  int64_t cap = static_cast<int64_t>(sm_count) * 8;
  int bx = static_cast<int>(blocks_needed < cap ? blocks_needed : cap);
  if (bx < 1) bx = 1;
  copy_chunks_kernel<<<dim3(bx, npairs), 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace dtb
