// Partial-attention forward for sm_100a: one launch computes, for every query row of a chunk, the
// softmax-attention state (out, lse) against ONE key/value chunk.
//
// CTA = 256 query rows of one (segment, head): two 128-row Q tiles that ping-pong on the tensor
// core.  Warp roles (320 threads):
//   warps 0-3   softmax group 0: one thread per row of Q tile 0
//   warps 4-7   softmax group 1: one thread per row of Q tile 1
//   warp  8     TMA producer: Q tiles once, then K_j, V_j tiles through a shared-memory ring
//   warp  9     MMA issuer (one elected thread): S_i = Q_i K_j^T and O_i += P_i V_j via tcgen05.mma
// Tensor memory (512 columns x 128 lanes of fp32): S_0 [0,128), S_1 [128,256), O_0 [256,256+D),
// O_1 [256+D,256+2D).  P_i (bf16) overwrites the first 64 columns of S_i and is consumed by the PV
// MMA straight from tensor memory.  Issue order on the tensor pipe:
//   S0(0) S1(0) | PV0(j) S0(j+1) PV1(j) S1(j+1) | ...
// so the softmax of one Q tile runs while the pipe works on the other tile.
// Running max is kept lazily: O is rescaled only when the max grew by more than 2^8, which bounds
// every probability by 2^8 and keeps bf16 P exact enough; the final normalisation undoes it.
#include "flash_fwd_sm100.cuh"
#include "ptx_sm100.cuh"

#include <math.h>

namespace dtb {

namespace {

constexpr int kBM = 128;        // query rows per tile
constexpr int kBN = 128;        // key rows per tile
constexpr int kQT = 2;          // query tiles per CTA
constexpr int kThreads = 320;
constexpr int kTmaWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kSlabBytes = 128 * 128;   // one TMA box: 128 rows x 64 bf16, 128-byte swizzled
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;   // log2 units

template <int D>
struct Cfg {
  static constexpr int kSlabs = D / 64;
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kStages = (D == 128) ? 4 : 6;
  static constexpr int kBars = 1 + 2 * kStages + 2 + 2 + 1;
  static constexpr int kSmemBytes = 1024 + (kQT + kStages) * kTileBytes + kBars * 8 + 16;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kColS = 0;      // + tile * 128
  static constexpr uint32_t kColO = 256;    // + tile * D
};

__device__ __forceinline__ void report(int* status, int code) {
  atomicCAS(status, 0, code);
}

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

__device__ __forceinline__ int64_t lse_index(const FlashParams& p, int seg, int head, int q_pos, int64_t tok) {
  if (p.lse_layout == 1) return tok * p.num_heads + head;                        // [B,S,H]
  if (p.cu_q != nullptr) return static_cast<int64_t>(head) * p.total_q + tok;    // [H,T]
  return (static_cast<int64_t>(seg) * p.num_heads + head) * p.seqlen_q + q_pos;  // [B,H,S]
}

}  // namespace

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const FlashParams p) {
  using C = Cfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem;
  uint8_t* s_kv = smem + kQT * C::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_kv + C::kStages * C::kTileBytes);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + C::kStages;
  uint64_t* s_full = kv_empty + C::kStages;
  uint64_t* p_full = s_full + 2;
  uint64_t* o_final = p_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::kBars);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int seg = blockIdx.z;
  const int head = blockIdx.y;

  int q_begin, q_len, k_begin, k_len;
  if (p.cu_q != nullptr) {
    q_begin = p.cu_q[seg];
    q_len = p.cu_q[seg + 1] - q_begin;
    k_begin = p.cu_k[seg];
    k_len = p.cu_k[seg + 1] - k_begin;
  } else {
    q_begin = seg * p.seqlen_q;
    q_len = p.seqlen_q;
    k_begin = seg * p.seqlen_k;
    k_len = p.seqlen_k;
  }
  const int q0 = blockIdx.x * (kQT * kBM);
  if (q0 >= q_len) return;
  const int n_tiles = (k_len + kBN - 1) / kBN;

  if (n_tiles <= 0) {
    // No keys: an empty state.  Merging an empty state into an accumulator changes nothing.
    if (!p.accumulate && warp < 8) {
      const int q_pos = q0 + threadIdx.x;
      if (q_pos < q_len) {
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
    }
    return;
  }

  // ------------------------------------------------------------------ set-up
  if (threadIdx.x == kTmaWarp * 32) {
    mbar_init(q_full, 1);
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], kBM);
    }
    mbar_init(o_final, 1);
    fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  // CTA-uniform view of the status word: a CTA that starts after a failure elsewhere does no work.
  const int aborted = __syncthreads_or(*reinterpret_cast<volatile int*>(p.status) != 0);
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (aborted) {
    // fall through to the tear-down
  } else if (warp == kTmaWarp) {
    // -------------------------------------------------------------- TMA producer
    if (elect_one()) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      mbar_expect_tx(q_full, kQT * C::kTileBytes);
      for (int t = 0; t < kQT; ++t)
        for (int s = 0; s < C::kSlabs; ++s)
          tma_load_2d(s_q + t * C::kTileBytes + s * kSlabBytes, &tm_q, q_full, head * D + s * 64,
                      q_begin + q0 + t * kBM);
      const int n_loads = 2 * n_tiles;     // K_0 V_0 K_1 V_1 ...
      for (int it = 0; it < n_loads; ++it) {
        const int stage = it % C::kStages;
        const int round = it / C::kStages;
        if (round > 0 && !wait_or_abort(&kv_empty[stage], (round - 1) & 1, p.status, 11)) break;
        mbar_expect_tx(&kv_full[stage], C::kTileBytes);
        const CUtensorMap* tm = (it & 1) ? &tm_v : &tm_k;
        const int row = k_begin + (it >> 1) * kBN;
        for (int s = 0; s < C::kSlabs; ++s)
          tma_load_2d(s_kv + stage * C::kTileBytes + s * kSlabBytes, tm, &kv_full[stage], head * D + s * 64, row);
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_qk = idesc_bf16_f32(kBM, kBN, false, false);
      constexpr uint32_t idesc_pv = idesc_bf16_f32(kBM, D, false, true);
      const uint32_t q_addr = smem_u32(s_q);
      const uint32_t kv_addr = smem_u32(s_kv);

      auto issue_s = [&](int tile, int stage) {
#pragma unroll
        for (int k16 = 0; k16 < D / 16; ++k16) {
          const uint32_t off = (k16 >> 2) * kSlabBytes + (k16 & 3) * 32;
          const uint64_t a = smem_desc_sw128(q_addr + tile * C::kTileBytes + off, 16, 1024);
          const uint64_t b = smem_desc_sw128(kv_addr + stage * C::kTileBytes + off, 16, 1024);
          mma_ss(tmem_base + C::kColS + tile * kBN, a, b, idesc_qk, k16 > 0);
        }
      };
      auto issue_pv = [&](int tile, int stage, bool acc) {
#pragma unroll
        for (int k16 = 0; k16 < kBN / 16; ++k16) {
          const uint64_t b = smem_desc_sw128(kv_addr + stage * C::kTileBytes + k16 * 2048, kSlabBytes, 1024);
          mma_ts(tmem_base + C::kColO + tile * D, tmem_base + C::kColS + tile * kBN + k16 * 8, b, idesc_pv,
                 (acc || k16 > 0) ? 1u : 0u);
        }
      };
      auto stage_of = [&](int it) { return it % C::kStages; };
      auto parity_of = [&](int it) { return static_cast<uint32_t>((it / C::kStages) & 1); };

      bool ok = wait_or_abort(q_full, 0, p.status, 21);
      if (ok) ok = wait_or_abort(&kv_full[stage_of(0)], parity_of(0), p.status, 22);
      if (ok) {
        tc_fence_after();
        issue_s(0, stage_of(0));
        mma_commit(&s_full[0]);
        issue_s(1, stage_of(0));
        mma_commit(&s_full[1]);
        mma_commit(&kv_empty[stage_of(0)]);
      }
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int it_v = 2 * j + 1, it_kn = 2 * j + 2;
        const bool more = (j + 1 < n_tiles);
        ok = wait_or_abort(&kv_full[stage_of(it_v)], parity_of(it_v), p.status, 23);
        if (!ok) break;
        ok = wait_or_abort(&p_full[0], j & 1, p.status, 24);
        if (!ok) break;
        tc_fence_after();
        issue_pv(0, stage_of(it_v), j > 0);
        if (more) {
          ok = wait_or_abort(&kv_full[stage_of(it_kn)], parity_of(it_kn), p.status, 25);
          if (!ok) break;
          tc_fence_after();
          issue_s(0, stage_of(it_kn));
          mma_commit(&s_full[0]);
        }
        ok = wait_or_abort(&p_full[1], j & 1, p.status, 26);
        if (!ok) break;
        tc_fence_after();
        issue_pv(1, stage_of(it_v), j > 0);
        mma_commit(&kv_empty[stage_of(it_v)]);
        if (more) {
          issue_s(1, stage_of(it_kn));
          mma_commit(&s_full[1]);
          mma_commit(&kv_empty[stage_of(it_kn)]);
        }
      }
      if (ok) mma_commit(o_final);
    }
    __syncwarp();
  } else {
    // -------------------------------------------------------------- softmax + epilogue
    const int tile = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t s_taddr = lane_base + C::kColS + tile * kBN;
    const uint32_t o_taddr = lane_base + C::kColO + tile * D;
    const float c = p.scale_log2;
    float m = -INFINITY;   // running max of raw scores (lazily updated)
    float l = 0.f;         // running sum of exp2((s - m) * c)
    bool ok = true;

    for (int j = 0; j < n_tiles; ++j) {
      ok = wait_or_abort(&s_full[tile], j & 1, p.status, 31 + tile);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[kBN];
#pragma unroll
      for (int q = 0; q < kBN / 32; ++q) tmem_ld32(s_taddr + q * 32, sr + q * 32);
      tmem_wait_ld();
      if (j == n_tiles - 1 && (k_len & (kBN - 1)) != 0) {
        const int valid = k_len - j * kBN;
#pragma unroll
        for (int i = 0; i < kBN; ++i)
          if (i >= valid) sr[i] = 0xff800000u;   // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < kBN; i += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(sr[i]));
        mx1 = fmaxf(mx1, __uint_as_float(sr[i + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(sr[i + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(sr[i + 3]));
      }
      const float m_new = fmaxf(fmaxf(m, fmaxf(mx0, mx1)), fmaxf(mx2, mx3));
      if (j == 0) {
        m = m_new;
      } else {
        const bool grow = (m_new - m) * c > kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
          // PV(j-1) of this tile has completed: the commit behind s_full covers it.
          const float f = ex2((m - m_new) * c);
#pragma unroll
          for (int q = 0; q < D / 32; ++q) {
            uint32_t orow[32];
            tmem_ld32(o_taddr + q * 32, orow);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * f);
            tmem_st32(o_taddr + q * 32, orow);
          }
          tmem_wait_st();
          l *= f;
          m = m_new;
        }
      }
      const float mc = m * c;
      float sum0 = 0.f, sum1 = 0.f;
      uint32_t pk[kBN / 2];
#pragma unroll
      for (int i = 0; i < kBN; i += 2) {
        const float p0 = ex2(fmaf(__uint_as_float(sr[i]), c, -mc));
        const float p1 = ex2(fmaf(__uint_as_float(sr[i + 1]), c, -mc));
        sum0 += p0;
        sum1 += p1;
        pk[i >> 1] = pack_bf16x2(p0, p1);
      }
      l += sum0 + sum1;
      tmem_st32(s_taddr, pk);
      tmem_st32(s_taddr + 32, pk + 32);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&p_full[tile]);
    }

    if (ok) ok = wait_or_abort(o_final, 0, p.status, 41);
    if (ok) {
      tc_fence_after();
      const int q_pos = q0 + tile * kBM + row;
      const bool valid = q_pos < q_len;
      const int64_t tok = static_cast<int64_t>(q_begin) + q_pos;
      const float lse_new = (m * c + log2f(l)) * kLn2;
      float w_new = 1.f / l;     // weight applied to the un-normalised O row
      float w_old = 0.f;
      int64_t li = 0;
      if (valid) {
        li = lse_index(p, seg, head, q_pos, tok);
        if (p.accumulate) {
          const float lse_old = p.lse[li];
          if (lse_old == -INFINITY) {
            p.lse[li] = lse_new;
          } else {
            const float mx = fmaxf(lse_old, lse_new);
            const float e_old = __expf(lse_old - mx), e_new = __expf(lse_new - mx);
            const float tot = e_old + e_new;
            p.lse[li] = mx + __logf(tot);
            w_old = e_old / tot;
            w_new = (e_new / tot) / l;
          }
        } else {
          p.lse[li] = lse_new;
        }
      }
#pragma unroll
      for (int q = 0; q < D / 32; ++q) {
        uint32_t orow[32];
        tmem_ld32(o_taddr + q * 32, orow);
        tmem_wait_ld();
        if (valid) {
          if (p.out_dtype == 0) {
            float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.out) + tok * p.out_tok_stride + head * D + q * 32);
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
            uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.out) + tok * p.out_tok_stride + head * D + q * 32);
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
      }
    }
  }

  // ------------------------------------------------------------------ tear-down
  if (*reinterpret_cast<volatile int*>(p.status) != 0) __nanosleep(1000000);   // let copies in flight land
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int D>
cudaError_t launch_flash(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FlashParams& p,
                         cudaStream_t stream) {
  using C = Cfg<D>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  dim3 grid((p.seqlen_q + kQT * kBM - 1) / (kQT * kBM), p.num_heads, p.nseg);
  flash_fwd_kernel<D><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, p);
  return cudaGetLastError();
}

template cudaError_t launch_flash<64>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const FlashParams&, cudaStream_t);
template cudaError_t launch_flash<128>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const FlashParams&, cudaStream_t);

}  // namespace dtb
