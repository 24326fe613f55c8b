// Partial-attention forward, one thread per query row: the kernel used at head dimension 128.
//
// CTA = 256 query rows of one (segment, head): two 128-row Q tiles share the tensor core.  Warp roles
// (320 threads):
//   warps 0-3   softmax group 0: one thread per row of Q tile 0
//   warps 4-7   softmax group 1: one thread per row of Q tile 1
//   warp  8     TMA producer: Q tiles once, then K_j, V_j tiles (64 keys each) through a shared-memory ring
//   warp  9     MMA issuer (one elected thread): S_i = Q_i K_j^T and O_i += P_i V_j via tcgen05.mma
// Tensor memory (512 columns x 128 lanes of fp32) is full at D = 128: per Q tile i two S buffers of 64 columns
// at [128 i, 128 i + 64) and [128 i + 64, 128 i + 128), and the O accumulators at [256 + D i, 256 + D i + D).
// S_i(j) sits in buffer j & 1 and P_i(j) (bf16) overwrites its first 32 columns.  S_i(j+2) is issued right
// behind PV_i(j) (the pipe runs MMAs in issue order, so P is read before it is overwritten), which means
// S_i(j+1) is already in tensor memory when the softmax group finishes tile j:
//     S0(0) S1(0) S0(1) S1(1) | PV0(j) S0(j+2) PV1(j) S1(j+2) | ...
// The price against 128-key tiles: twice as many S instructions, and Q is re-read from shared memory per 64
// keys instead of per 128.
//
// Exp turns: warp w of group 0 and warp w of group 1 sit on the same scheduler and feed the same ex2 unit
// (16 results per clock per SM; 64 keys x 256 rows need 1024 clocks, exactly what the MMAs of the same step
// need).  They alternate in the exp phase through `exp_turn` barriers, so one warp's tensor-memory loads, row
// max and waits overlap the other's ex2 stream instead of both streams running side by side at half rate.
// Every hand-over (P to the issuer, the turn to the sibling) is one arrival per warp.
//
// Running max is kept lazily: O is rescaled only when the max grew by more than 2^8, which bounds every
// probability by 2^8 and keeps bf16 P exact enough; the final normalisation undoes it.
#include "flash_common.cuh"

#include <mutex>

namespace dtb {

namespace {

using namespace flash;

constexpr int kThreads = 320;
constexpr int kTmaWarp = 8;
constexpr int kMmaWarp = 9;

template <int D>
struct Cfg {
  static constexpr int kSlabs = D / 64;
  static constexpr int kTileBytes = kBM * D * 2;          // one Q tile
  static constexpr int kKvTileBytes = kBN * D * 2;        // one K or V tile
  static constexpr int kStages = 8;
  // barriers: q_full, kv_full[S], kv_empty[S], s_full[4], p_full[4], pv_done[2], exp_turn[8], o_final
  static constexpr int kBars = 1 + 2 * kStages + 4 + 4 + 2 + 8 + 1;
  static constexpr int kSmemBytes = 1024 + kQT * kTileBytes + kStages * kKvTileBytes + kBars * 8 + 16;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kColS = 0;          // + tile * 128 + buffer * 64
  static constexpr uint32_t kColO = 256;        // + tile * D
  static_assert(kColO + kQT * D <= 512, "tensor memory");
};

#ifdef DTB_FLASH_TIMING
// softmax phases: 0 before the wait for S, 1 S ready, 2 row max known, 3 rescale decided, 4 exp turn acquired,
//                 5 exp loop done, 6 P handed over;
// issuer phases:  0 top of step, 1 V ready, 2 P0 ready, 3 PV0 + S0(j+2) issued, 4 P1 ready, 5 PV1 + S1(j+2) issued.
__device__ long long g_timing_row[3 * 48 * 8];
#endif
#define STAMP(role, j, phase) DTB_STAMP(g_timing_row, role, j, phase)

}  // namespace

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
flash_fwd_row_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const FlashParams p) {
  using C = Cfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem;
  uint8_t* s_kv = smem + kQT * C::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_kv + C::kStages * C::kKvTileBytes);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + C::kStages;
  uint64_t* s_full = kv_empty + C::kStages;   // [tile*2 + buffer]: S_tile(j) is in tensor memory
  uint64_t* p_full = s_full + 4;              // [tile*2 + buffer]: P_tile(j) written (one arrival per softmax warp)
  uint64_t* pv_done = p_full + 4;             // [tile]: PV_tile(j) has completed
  uint64_t* exp_turn = pv_done + 2;           // [tile*4 + quarter]: the sibling warp finished its exp phase
  uint64_t* o_final = exp_turn + 8;
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
    grid_dependency_wait();      // (also when nothing is written: a grid must not complete before the one it overlaps)
    write_empty_rows<D>(p, seg, head, q_begin, q_len, q0);
    return;
  }

  // Position of K_j / V_j in the order the ring carries them: K_0 K_1 V_0 K_2 V_1 ... K_{n-1} V_{n-2} V_{n-1}
  // (K_{j+2} follows V_j, as S(j+2) follows PV(j) on the pipe).
  auto k_slot = [&](int j) { return j < 2 ? j : 2 * j - 1; };
  auto v_slot = [&](int j) { return j < n_tiles - 1 ? 2 * j + 2 : 2 * j + 1; };

  // ------------------------------------------------------------------ set-up
  if (threadIdx.x == kTmaWarp * 32) {
    mbar_init(q_full, 1);
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
    }
    for (int i = 0; i < 2; ++i) mbar_init(&pv_done[i], 1);
    for (int i = 0; i < 8; ++i) mbar_init(&exp_turn[i], 1);
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
  // From here on a launch queued behind this one with the overlap attribute may fill idle SMs (it takes effect
  // once every CTA of this grid has got this far); it waits for this grid's completion before it touches results.
  grid_launch_dependents();
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
      const int n_loads = 2 * n_tiles;
      for (int it = 0; it < n_loads; ++it) {
        bool is_v;
        int j;
        if (it == n_loads - 1) { is_v = true; j = n_tiles - 1; }
        else if (it < 2) { is_v = false; j = it; }
        else if (it & 1) { is_v = false; j = (it + 1) >> 1; }
        else { is_v = true; j = (it - 2) >> 1; }
        const int stage = it % C::kStages;
        const int round = it / C::kStages;
        if (round > 0 && !wait_or_abort(&kv_empty[stage], (round - 1) & 1, p.status, 11)) break;
        mbar_expect_tx(&kv_full[stage], C::kKvTileBytes);
        const CUtensorMap* tm = is_v ? &tm_v : &tm_k;
        const int row = k_begin + j * kBN;
        for (int s = 0; s < C::kSlabs; ++s)
          tma_load_2d(s_kv + stage * C::kKvTileBytes + s * kKvSlabBytes, tm, &kv_full[stage], head * D + s * 64, row);
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

      // Descriptors are built once; a tile, stage or K step only moves the start-address field (units
      // of 16 bytes, no carry out of the field: shared memory ends below 2^18).
      const uint64_t q_desc = smem_desc_sw128(q_addr, 16, 1024);               // K-major
      const uint64_t k_desc = smem_desc_sw128(kv_addr, 16, 1024);              // K-major
      const uint64_t v_desc = smem_desc_sw128(kv_addr, kKvSlabBytes, 1024);    // MN-major, slab pitch leading
      // S_tile = Q_tile K^T into S columns [128 tile + s_col, ... + 64)
      auto issue_s = [&](int tile, int stage, int s_col) {
        const uint64_t a0 = q_desc + static_cast<uint32_t>(tile * (C::kTileBytes >> 4));
        const uint64_t b0 = k_desc + static_cast<uint32_t>(stage * (C::kKvTileBytes >> 4));
        const uint32_t d = tmem_base + C::kColS + tile * 128 + s_col;
#pragma unroll
        for (int k16 = 0; k16 < D / 16; ++k16) {
          const uint32_t in_slab = (k16 & 3) * 32;
          mma_ss(d, a0 + (((k16 >> 2) * kSlabBytes + in_slab) >> 4), b0 + (((k16 >> 2) * kKvSlabBytes + in_slab) >> 4),
                 idesc_qk, k16 > 0);
        }
      };
      // O_tile (+)= P_tile V: four K=16 steps over the 64 keys, P (bf16 pairs) at tensor-memory column p_col
      auto issue_pv = [&](int tile, int stage, bool acc, uint32_t p_col) {
        const uint64_t b0 = v_desc + static_cast<uint32_t>(stage * (C::kKvTileBytes >> 4));
        const uint32_t d = tmem_base + C::kColO + tile * D;
        const uint32_t a = tmem_base + p_col;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_ts(d, a + kk * 8, b0 + (kk * 2048 >> 4), idesc_pv, (acc || kk > 0) ? 1u : 0u);
      };
      auto stage_of = [&](int it) { return it % C::kStages; };
      auto parity_of = [&](int it) { return static_cast<uint32_t>((it / C::kStages) & 1); };
      auto wait_kv = [&](int it, int code) {
        return wait_or_abort(&kv_full[stage_of(it)], parity_of(it), p.status, code);
      };

      bool ok = wait_or_abort(q_full, 0, p.status, 21);
      // S(0) and S(1) of both Q tiles fill the two buffers; from then on S(j+2) follows PV(j).
      for (int j = 0; ok && j < 2 && j < n_tiles; ++j) {
        ok = wait_kv(k_slot(j), 22);
        if (!ok) break;
        tc_fence_after();
        for (int tile = 0; tile < 2; ++tile) {
          issue_s(tile, stage_of(k_slot(j)), j * kBN);
          mma_commit(&s_full[tile * 2 + j]);
        }
        mma_commit(&kv_empty[stage_of(k_slot(j))]);
      }
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int buf = j & 1;
        const bool more = (j + 2 < n_tiles);
        const int it_v = v_slot(j), it_kn = k_slot(j + 2);
        STAMP(2, j, 0);
        ok = wait_kv(it_v, 23);
        if (!ok) break;
        STAMP(2, j, 1);
        for (int tile = 0; tile < 2; ++tile) {
          ok = wait_or_abort(&p_full[tile * 2 + buf], (j >> 1) & 1, p.status, 24 + tile);
          if (!ok) break;
          STAMP(2, j, 2 + 2 * tile);
          tc_fence_after();
          issue_pv(tile, stage_of(it_v), j > 0, C::kColS + tile * 128 + buf * kBN);
          mma_commit(&pv_done[tile]);
          if (tile == 1) mma_commit(&kv_empty[stage_of(it_v)]);
          if (more) {
            if (tile == 0) {
              ok = wait_kv(it_kn, 25);
              if (!ok) break;
              tc_fence_after();
            }
            // overwrites P_tile(j); the pipe runs it behind PV_tile(j)
            issue_s(tile, stage_of(it_kn), buf * kBN);
            mma_commit(&s_full[tile * 2 + buf]);
            if (tile == 1) mma_commit(&kv_empty[stage_of(it_kn)]);
          }
          STAMP(2, j, 3 + 2 * tile);
        }
      }
      if (ok) mma_commit(o_final);
    }
    __syncwarp();
  } else {
    // -------------------------------------------------------------- softmax + epilogue
    const int tile = warp >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_taddr = lane_base + C::kColS + tile * 128;
    const uint32_t o_taddr = lane_base + C::kColO + tile * D;
    const float c = p.scale_log2;
    float m = -INFINITY;   // running max of raw scores (lazily updated)
    float l = 0.f;         // running sum of exp2((s - m) * c)
    bool ok = true;
    const bool stamp = (lane == 0 && quarter == 0);
    (void)stamp;

    for (int j = 0; j < n_tiles; ++j) {
      const int buf = j & 1;
      const uint32_t sb_taddr = s_taddr + buf * kBN;   // S_tile(j), then P_tile(j) over its first half
      if (stamp) STAMP(tile, j, 0);
      ok = wait_or_abort(&s_full[tile * 2 + buf], (j >> 1) & 1, p.status, 31 + tile);
      if (!ok) break;
      if (stamp) STAMP(tile, j, 1);
      tc_fence_after();
      uint32_t sr[kBN];
      tmem_ld32(sb_taddr, sr);
      tmem_ld32(sb_taddr + 32, sr + 32);
      tmem_wait_ld();
      if ((j == n_tiles - 1) && (k_len & (kBN - 1)) != 0) {
        const int valid = k_len - j * kBN;
#pragma unroll
        for (int i = 0; i < kBN; ++i)
          if (i >= valid) sr[i] = 0xff800000u;   // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < kBN; i += 8) {
        mx0 = max3(mx0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
        mx1 = max3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
        mx2 = max3(mx2, __uint_as_float(sr[i + 4]), __uint_as_float(sr[i + 5]));
        mx3 = max3(mx3, __uint_as_float(sr[i + 6]), __uint_as_float(sr[i + 7]));
      }
      if (stamp) STAMP(tile, j, 2);
      const float m_new = fmaxf(max3(m, mx0, mx1), fmaxf(mx2, mx3));
      if (j == 0) {
        m = m_new;
      } else {
        const bool grow = (m_new - m) * c > kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
          // O is rescaled in place: PV_tile(j-1) must have drained (PV_tile(j) is not issued before
          // this group hands over P_tile(j), so nothing else is in flight on O)
          ok = wait_or_abort(&pv_done[tile], (j - 1) & 1, p.status, 33 + tile);
          if (!ok) break;
          tc_fence_after();
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
      if (stamp) STAMP(tile, j, 3);
      // The turn: groups alternate 0, 1, 0, 1, ...; group 0's first turn is free (parity trick).
      ok = wait_or_abort(&exp_turn[tile * 4 + quarter], tile == 0 ? ((j & 1) ^ 1) : (j & 1), p.status, 35 + tile);
      if (!ok) break;
      if (stamp) STAMP(tile, j, 4);
      // p = 2^(s*c - m*c): one ex2 per score against 4*D tensor FLOPs per score
      const float nmc = -m * c;
      float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
      uint32_t pk[kBN / 2];
#pragma unroll
      for (int g = 0; g < kBN / 8; ++g) {
#pragma unroll
        for (int pr = 0; pr < 4; ++pr) {
          const int i = g * 8 + pr * 2;
          const float p0 = ex2(fmaf(__uint_as_float(sr[i]), c, nmc));
          const float p1 = ex2(fmaf(__uint_as_float(sr[i + 1]), c, nmc));
          if (pr & 1) {
            sum2 += p0;
            sum3 += p1;
          } else {
            sum0 += p0;
            sum1 += p1;
          }
          pk[i >> 1] = pack_bf16x2(p0, p1);
        }
      }
      if (stamp) STAMP(tile, j, 5);
      tmem_st32(sb_taddr, pk);
      tmem_wait_st();
      tc_fence_before();
      // One arrival per warp for both hand-overs.  Passing the turn on any earlier (after the exp loop, or
      // part-way through it) was measured 10 % slower: the two groups then drift into phase and exponentiate
      // side by side.
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&p_full[tile * 2 + buf]);
        mbar_arrive(&exp_turn[(tile ^ 1) * 4 + quarter]);
      }
      if (stamp) STAMP(tile, j, 6);
      l += (sum0 + sum1) + (sum2 + sum3);
    }

    if (ok) ok = wait_or_abort(o_final, 0, p.status, 41);
    // Results: the launch before this one (which may still be running if this launch overlaps it) must have
    // completed before its state is read for accumulation or its buffers are written.
    grid_dependency_wait();
    if (ok) {
      tc_fence_after();
      const int q_pos = q0 + tile * kBM + row;
      const bool valid = q_pos < q_len;
      const int64_t tok = static_cast<int64_t>(q_begin) + q_pos;
      const float lse_new = (m * c + log2f(l)) * kLn2;
      float w_new = 1.f / l, w_old = 0.f;
      if (valid) {
        const int64_t li = lse_index(p, seg, head, q_pos, tok);
        float lse_out;
        merge_weights(p.accumulate != 0, p.accumulate ? p.lse[li] : -INFINITY, lse_new, l, w_new, w_old, lse_out);
        p.lse[li] = lse_out;
      }
#pragma unroll
      for (int q = 0; q < D / 32; ++q) {
        uint32_t orow[32];
        tmem_ld32(o_taddr + q * 32, orow);
        tmem_wait_ld();
        if (valid) store_row_chunk32(p, tok, static_cast<int64_t>(head) * D + q * 32, orow, w_new, w_old);
      }
    }
  }

  // ------------------------------------------------------------------ tear-down
  // No CTA leaves before the launch it may overlap has completed: a launch that overlaps THIS one waits for this
  // grid only, and relies on this grid's completion implying that of everything before it.
  grid_dependency_wait();
  if (*reinterpret_cast<volatile int*>(p.status) != 0) __nanosleep(1000000);   // let copies in flight land
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int D>
cudaError_t launch_flash_row(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FlashParams& p,
                             cudaStream_t stream) {
  using C = Cfg<D>;
  static bool configured[64] = {};
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64) {
    std::lock_guard<std::mutex> lk(mu);
    if (!configured[dev]) {
      cudaError_t e = cudaFuncSetAttribute(flash_fwd_row_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
      if (e != cudaSuccess) return e;
      configured[dev] = true;
    }
  }
  dim3 grid((p.seqlen_q + kQT * kBM - 1) / (kQT * kBM), p.num_heads, p.nseg);
  return launch_attention_kernel(flash_fwd_row_kernel<D>, grid, kThreads, C::kSmemBytes, stream, p.overlap_previous != 0, tq, tk, tv, p);
}

#ifdef DTB_FLASH_TIMING
cudaError_t read_flash_timing_row(long long* host, int n) {
  return cudaMemcpyFromSymbol(host, g_timing_row, sizeof(long long) * n);
}
#endif

template cudaError_t launch_flash_row<128>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const FlashParams&, cudaStream_t);

}  // namespace dtb
