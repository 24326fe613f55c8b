// Pieces shared by the two partial-attention forward kernels (flash_fwd_row.cu: one thread per query row,
// flash_fwd_pair.cu: two threads per query row): tile geometry, the bounded barrier wait, the status word,
// packed fp32 arithmetic, the lse layouts, and the development-time phase stamps.
#pragma once
#include "flash_fwd_sm100.cuh"
#include "ptx_sm100.cuh"

#include <math.h>

namespace dtb {
namespace flash {

constexpr int kBM = 128;                  // query rows per tile
constexpr int kQT = 2;                    // query tiles per CTA
constexpr int kBN = 64;                   // key rows per tile
constexpr int kSlabBytes = 128 * 128;     // one TMA box of Q: 128 rows x 64 bf16, 128-byte swizzled
constexpr int kKvSlabBytes = kBN * 128;   // one TMA box of K / V: 64 rows x 64 bf16
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f; // log2 units: the running reference follows the maximum this lazily

__device__ __forceinline__ void report(int* status, int code) { atomicCAS(status, 0, code); }

// Bounded wait that also gives up as soon as any CTA has reported a failure.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (((++spins) & 0xff) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;
      if (globaltimer_ns() - t0 > 1000000000ull) {
        report(status, code);
        return false;
      }
    }
  }
  return true;
}

// ---------------------------------------------------------------------------- packed fp32 pairs
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

__device__ __forceinline__ int64_t lse_index(const FlashParams& p, int seg, int head, int q_pos, int64_t tok) {
  if (p.lse_layout == 1) return tok * p.num_heads + head;                        // [B,S,H]
  if (p.cu_q != nullptr) return static_cast<int64_t>(head) * p.total_q + tok;    // [H,T]
  return (static_cast<int64_t>(seg) * p.num_heads + head) * p.seqlen_q + q_pos;  // [B,H,S]
}

// Rows of a (segment, head) that has no keys at all: an empty state (out = 0, lse = -inf).  Merging an empty
// state into an accumulator changes nothing, so with accumulate set nothing is written.  The first 256
// threads of the CTA cover its 256 query rows.
template <int D>
__device__ __forceinline__ void write_empty_rows(const FlashParams& p, int seg, int head, int q_begin, int q_len, int q0) {
  if (p.accumulate || threadIdx.x >= kQT * kBM) return;
  const int q_pos = q0 + threadIdx.x;
  if (q_pos >= q_len) return;
  grid_dependency_wait();      // the launch before this one may still be writing the same buffers
  const int64_t tok = static_cast<int64_t>(q_begin) + q_pos;
  p.lse[lse_index(p, seg, head, q_pos, tok)] = -INFINITY;
  if (p.out_dtype == 0) {
    float4* o = reinterpret_cast<float4*>(static_cast<float*>(p.out) + tok * p.out_tok_stride + head * D);
    for (int c = 0; c < D / 4; ++c) o[c] = make_float4(0.f, 0.f, 0.f, 0.f);
  } else {
    uint4* o = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out) + tok * p.out_tok_stride + head * D);
    for (int c = 0; c < D / 8; ++c) o[c] = make_uint4(0u, 0u, 0u, 0u);
  }
}

// Final step for 32 consecutive columns of one output row held in `orow` (un-normalised fp32 accumulators):
// scale by w_new, blend with the state already in global memory when accumulating (w_old != 0), store as
// fp32 or bf16.  `col` is the element offset of the 32 columns inside the row's token.
__device__ __forceinline__ void store_row_chunk32(const FlashParams& p, int64_t tok, int64_t col, const uint32_t (&orow)[32],
                                                  float w_new, float w_old) {
  if (p.out_dtype == 0) {
    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.out) + tok * p.out_tok_stride + col);
    if (p.accumulate && w_old != 0.f) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float4 o = dst[i];
        o.x = o.x * w_old + __uint_as_float(orow[4 * i]) * w_new;
        o.y = o.y * w_old + __uint_as_float(orow[4 * i + 1]) * w_new;
        o.z = o.z * w_old + __uint_as_float(orow[4 * i + 2]) * w_new;
        o.w = o.w * w_old + __uint_as_float(orow[4 * i + 3]) * w_new;
        dst[i] = o;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        dst[i] = make_float4(__uint_as_float(orow[4 * i]) * w_new, __uint_as_float(orow[4 * i + 1]) * w_new,
                             __uint_as_float(orow[4 * i + 2]) * w_new, __uint_as_float(orow[4 * i + 3]) * w_new);
    }
  } else {
    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out) + tok * p.out_tok_stride + col);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 v;
      v.x = pack_bf16x2(__uint_as_float(orow[8 * i]) * w_new, __uint_as_float(orow[8 * i + 1]) * w_new);
      v.y = pack_bf16x2(__uint_as_float(orow[8 * i + 2]) * w_new, __uint_as_float(orow[8 * i + 3]) * w_new);
      v.z = pack_bf16x2(__uint_as_float(orow[8 * i + 4]) * w_new, __uint_as_float(orow[8 * i + 5]) * w_new);
      v.w = pack_bf16x2(__uint_as_float(orow[8 * i + 6]) * w_new, __uint_as_float(orow[8 * i + 7]) * w_new);
      dst[i] = v;
    }
  }
}

// Weights of the final normalisation: a row whose un-normalised accumulator has row sum l_row and log-sum-exp
// lse_new is either written as is (w_new = 1 / l_row) or merged with the state (lse_old) already in memory.
__device__ __forceinline__ void merge_weights(bool accumulate, float lse_old, float lse_new, float l_row, float& w_new,
                                              float& w_old, float& lse_out) {
  w_new = 1.f / l_row;
  w_old = 0.f;
  lse_out = lse_new;
  if (accumulate && lse_old != -INFINITY) {
    const float mx = fmaxf(lse_old, lse_new);
    const float e_old = __expf(lse_old - mx), e_new = __expf(lse_new - mx);
    const float tot = e_old + e_new;
    lse_out = mx + __logf(tot);
    w_old = e_old / tot;
    w_new = (e_new / tot) / l_row;
  }
}

// Host: one launch of an attention kernel, with the programmatic-stream-serialization attribute when the caller
// allows the launch to overlap the end of the one before it.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_attention_kernel(void (*kernel)(KArgs...), dim3 grid, int threads, size_t smem_bytes,
                                           cudaStream_t stream, bool overlap_previous, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap_previous ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Args&&>(args)...);
}

}  // namespace flash

#ifdef DTB_FLASH_TIMING
// Development aid: per-phase SM clock stamps of one CTA, timing[role][key tile j < 48][phase], read back with
// dtb_debug_flash_timing (exported only in this build).  Roles 0, 1: first softmax warp of each Q tile;
// role 2: the MMA issuer.
#define DTB_STAMP(table, role, j, phase)                                                               \
  do {                                                                                                 \
    if (blockIdx.x == 1 && blockIdx.y == 0 && blockIdx.z == 0 && (j) < 48)                             \
      table[((role) * 48 + (j)) * 8 + (phase)] = clock64();                                            \
  } while (0)
#else
#define DTB_STAMP(table, role, j, phase) do { } while (0)
#endif

}  // namespace dtb
