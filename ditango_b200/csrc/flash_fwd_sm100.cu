// Partial-attention forward for sm_100a: one launch computes, for every query row of a chunk, the
// softmax-attention state (out, lse) against ONE key/value chunk.
//
// CTA = 256 query rows of one (segment, head): two 128-row Q tiles share the tensor core.  Warp roles
// (320 threads):
//   warps 0-3   softmax group 0: one thread per row of Q tile 0
//   warps 4-7   softmax group 1: one thread per row of Q tile 1
//   warp  8     TMA producer: Q tiles once, then K_j, V_j tiles through a shared-memory ring
//   warp  9     MMA issuer (one elected thread): S_i = Q_i K_j^T and O_i += P_i V_j via tcgen05.mma
// Tensor memory (512 columns x 128 lanes of fp32): S_0 [0,128), S_1 [128,256), O_0 [256,256+D),
// O_1 [256+D,256+2D).  Three schedules, chosen at compile time by what fits:
//   D = 64 ("decoupled"): 128 columns are left, so P_i (bf16) gets its own columns [384 + 64 i,
//     448 + 64 i).  Key tiles of 128 rows; S_i(j+1) is issued as soon as the softmax group has pulled
//     S_i(j) into registers, ahead of PV_i(j):
//       S0(0) S1(0) | S0(j+1) S1(j+1) PV0(j) PV1(j) | ...
//     and in steady state a softmax group never waits for the tensor pipe.  P is handed to the MMA
//     issuer in two halves (keys 0-63, 64-127) so the first PV steps start while the second half is
//     still being exponentiated.
//   D = 128 ("split", DTB_SPLIT_KV=1, the default): the map is full.  Key tiles of 64 rows and two S
//     buffers of 64 columns per Q tile: S_i(j) sits in buffer j & 1 and P_i(j) overwrites its first 32
//     columns.  S_i(j+2) follows PV_i(j) on the pipe, so S_i(j+1) is already there when a softmax
//     group finishes tile j:
//       S0(0) S1(0) S0(1) S1(1) | PV0(j) S0(j+2) PV1(j) S1(j+2) | ...
//     The price: twice as many S instructions, and Q is re-read from shared memory per 64 keys instead
//     of per 128 (the data banks stay under 30 % busy).
//   D = 128 ("coupled", DTB_SPLIT_KV=0): key tiles of 128 rows, P_i over the first 64 columns of S_i,
//       S0(0) S1(0) | PV0(j) S0(j+1) PV1(j) S1(j+1) | ...
//     each Q tile runs the serial chain softmax -> PV -> next S; only the other tile's work overlaps.
// Running max is kept lazily: O is rescaled only when the max grew by more than 2^8, which bounds
// every probability by 2^8 and keeps bf16 P exact enough; the final normalisation undoes it.
#include "flash_fwd_sm100.cuh"
#include "ptx_sm100.cuh"

#include <math.h>

#include <mutex>

namespace dtb {

namespace {

#ifndef DTB_SPLIT_KV
#define DTB_SPLIT_KV 1
#endif
#ifndef DTB_SPLIT_TURNS
#define DTB_SPLIT_TURNS 1
#endif

constexpr int kBM = 128;        // query rows per tile
constexpr int kQT = 2;          // query tiles per CTA
constexpr int kThreads = 320;
constexpr int kTmaWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kSlabBytes = 128 * 128;   // one TMA box of Q: 128 rows x 64 bf16, 128-byte swizzled
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;   // log2 units

template <int D>
struct Cfg {
  static constexpr int kSlabs = D / 64;
  // 64-key tiles with double-buffered S (see the head of this file)
  static constexpr bool kSplit = (D == 128) && (DTB_SPLIT_KV != 0);
  static constexpr int kBN = kSplit ? 64 : 128;          // key rows per tile
  static constexpr int kTileBytes = 128 * D * 2;         // one Q tile
  static constexpr int kKvTileBytes = kBN * D * 2;       // one K or V tile
  static constexpr int kKvSlabBytes = kBN * 128;         // one TMA box of K / V: kBN rows x 64 bf16
  static constexpr int kStages = kSplit ? 8 : ((D == 128) ? 4 : 6);
  // P in its own tensor-memory columns and S_i(j+1) issued ahead of PV_i(j)
  static constexpr bool kDecoupled = !kSplit && (256 + 2 * D + 128 <= 512);
  // sibling warps of the two softmax groups alternate in the exp phase
  static constexpr bool kTurns = kDecoupled || (kSplit && DTB_SPLIT_TURNS != 0);
  // of every 4 score pairs, this many take the polynomial exp2 instead of the ex2 unit
#ifdef DTB_EMU_PAIRS
  static constexpr int kEmuPairs = DTB_EMU_PAIRS;
#else
  static constexpr int kEmuPairs = 0;
#endif
  // barriers: q_full, kv_full[S], kv_empty[S], s_full[4], p_full[4], s_free[2], pv_done[2], exp_turn[8], o_final
  static constexpr int kBars = 1 + 2 * kStages + 4 + 4 + 2 + 2 + 8 + 1;
  static constexpr int kSmemBytes = 1024 + kQT * kTileBytes + kStages * kKvTileBytes + kBars * 8 + 16;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kColS = 0;                                  // + tile * 128
  static constexpr uint32_t kColO = 256;                                // + tile * D
  static constexpr uint32_t kColP = kDecoupled ? 256 + 2 * D : 0;       // + tile * kStrideP
  static constexpr uint32_t kStrideP = kDecoupled ? 64 : 128;
};

#ifdef DTB_FLASH_TIMING
// Development aid: per-phase SM clock stamps of one CTA, g_flash_timing[role][key tile j < 48][phase],
// read back with dtb_debug_flash_timing (exported only in this build).  Roles 0, 1: first warp of each
// softmax group; role 2: the MMA issuer.  Phases of the split schedule --
//   softmax: 0 before the wait for S, 1 S ready, 2 row max known, 3 rescale decided, 4 exp turn acquired,
//            5 exp loop done, 6 P handed over;
//   issuer:  0 top of step, 1 V ready, 2 P0 ready, 3 PV0 + S0(j+2) issued, 4 P1 ready, 5 PV1 + S1(j+2) issued.
__device__ long long g_flash_timing[3 * 48 * 8];
#define DTB_STAMP(role, j, phase)                                                                      \
  do {                                                                                                 \
    if (blockIdx.x == 1 && blockIdx.y == 0 && blockIdx.z == 0 && (j) < 48)                             \
      g_flash_timing[((role) * 48 + (j)) * 8 + (phase)] = clock64();                                   \
  } while (0)
#else
#define DTB_STAMP(role, j, phase) do { } while (0)
#endif

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

// 2^x for a pair of fp32 values without the ex2 unit: x is clamped to >= -126, split as n + f with
// n = round(x) (magic-number add) and f in [-0.5, 0.5], 2^f by a cubic (max relative error 7.5e-5,
// far below the bf16 rounding of P), and n added into the exponent field.
__device__ __forceinline__ void exp2_poly_pair(float x0, float x1, float& p0, float& p1) {
  x0 = fmaxf(x0, -126.f);
  x1 = fmaxf(x1, -126.f);
  const float t0 = x0 + 12582912.f, t1 = x1 + 12582912.f;
  const float f0 = x0 - (t0 - 12582912.f), f1 = x1 - (t1 - 12582912.f);
  float q0 = fmaf(0.0551716685f, f0, 0.2426111251f), q1 = fmaf(0.0551716685f, f1, 0.2426111251f);
  q0 = fmaf(q0, f0, 0.6932609677f);
  q1 = fmaf(q1, f1, 0.6932609677f);
  q0 = fmaf(q0, f0, 0.9999280572f);
  q1 = fmaf(q1, f1, 0.9999280572f);
  p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
  p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
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
  constexpr int kBN = C::kBN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem;
  uint8_t* s_kv = smem + kQT * C::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_kv + C::kStages * C::kKvTileBytes);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + C::kStages;
  uint64_t* s_full = kv_empty + C::kStages;   // [tile] (split: [tile*2 + buffer]): S_tile(j) is in tensor memory
  uint64_t* p_full = s_full + 4;              // [tile*2 + half]: P of keys [64 half, 64 half + 64) written
                                              // (split: [tile*2 + buffer], the whole 64-key tile)
  uint64_t* s_free = p_full + 4;              // [tile]: S_tile(j) has been read into registers (decoupled)
  uint64_t* pv_done = s_free + 2;             // [tile]: PV_tile(j) has completed (decoupled)
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

  // Position of K_j / V_j in the order the ring carries them.
  //   coupled:   K_0 V_0 K_1 V_1 ...                 (K_j at 2j, V_j at 2j+1)
  //   decoupled: K_0 K_1 V_0 K_2 V_1 ... V_{n-1}     (K_{j+1} is consumed before V_j)
  //   split:     K_0 K_1 V_0 K_2 V_1 ... K_{n-1} V_{n-2} V_{n-1}   (K_{j+2} follows V_j)
  auto k_slot = [&](int j) {
    if (C::kSplit) return j < 2 ? j : 2 * j - 1;
    return C::kDecoupled ? (j == 0 ? 0 : 2 * j - 1) : 2 * j;
  };
  auto v_slot = [&](int j) {
    if (C::kSplit) return j < n_tiles - 1 ? 2 * j + 2 : 2 * j + 1;
    return C::kDecoupled ? (j < n_tiles - 1 ? 2 * j + 2 : 2 * j + 1) : 2 * j + 1;
  };

  // ------------------------------------------------------------------ set-up
  if (threadIdx.x == kTmaWarp * 32) {
    mbar_init(q_full, 1);
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&s_full[i], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_free[i], kBM);
      mbar_init(&pv_done[i], 1);
    }
    for (int i = 0; i < 8; ++i) mbar_init(&exp_turn[i], 32);
    for (int i = 0; i < 4; ++i) mbar_init(&p_full[i], kBM);
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
      const int n_loads = 2 * n_tiles;
      for (int it = 0; it < n_loads; ++it) {
        bool is_v;
        int j;
        if (C::kSplit) {
          if (it == n_loads - 1) { is_v = true; j = n_tiles - 1; }
          else if (it < 2) { is_v = false; j = it; }
          else if (it & 1) { is_v = false; j = (it + 1) >> 1; }
          else { is_v = true; j = (it - 2) >> 1; }
        } else if (C::kDecoupled) {
          if (it == 0) { is_v = false; j = 0; }
          else if (it == n_loads - 1) { is_v = true; j = n_tiles - 1; }
          else if (it & 1) { is_v = false; j = (it + 1) >> 1; }
          else { is_v = true; j = (it - 2) >> 1; }
        } else {
          is_v = it & 1;
          j = it >> 1;
        }
        const int stage = it % C::kStages;
        const int round = it / C::kStages;
        if (round > 0 && !wait_or_abort(&kv_empty[stage], (round - 1) & 1, p.status, 11)) break;
        mbar_expect_tx(&kv_full[stage], C::kKvTileBytes);
        const CUtensorMap* tm = is_v ? &tm_v : &tm_k;
        const int row = k_begin + j * kBN;
        for (int s = 0; s < C::kSlabs; ++s)
          tma_load_2d(s_kv + stage * C::kKvTileBytes + s * C::kKvSlabBytes, tm, &kv_full[stage], head * D + s * 64, row);
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
      const uint64_t q_desc = smem_desc_sw128(q_addr, 16, 1024);                  // K-major
      const uint64_t k_desc = smem_desc_sw128(kv_addr, 16, 1024);                 // K-major
      const uint64_t v_desc = smem_desc_sw128(kv_addr, C::kKvSlabBytes, 1024);    // MN-major, slab pitch leading
      // S_tile = Q_tile K^T into S columns [128 tile + s_col, ... + kBN)
      auto issue_s = [&](int tile, int stage, int s_col = 0) {
        const uint64_t a0 = q_desc + static_cast<uint32_t>(tile * (C::kTileBytes >> 4));
        const uint64_t b0 = k_desc + static_cast<uint32_t>(stage * (C::kKvTileBytes >> 4));
        const uint32_t d = tmem_base + C::kColS + tile * 128 + s_col;
#pragma unroll
        for (int k16 = 0; k16 < D / 16; ++k16) {
          const uint32_t in_slab = (k16 & 3) * 32;
          mma_ss(d, a0 + (((k16 >> 2) * kSlabBytes + in_slab) >> 4), b0 + (((k16 >> 2) * C::kKvSlabBytes + in_slab) >> 4),
                 idesc_qk, k16 > 0);
        }
      };
      // half h covers keys [64 h, 64 h + 64) of the tile: four K=16 steps of P (at column p_col) times V
      auto issue_pv = [&](int tile, int stage, int half, bool acc, uint32_t p_col) {
        const uint64_t b0 = v_desc + static_cast<uint32_t>(stage * (C::kKvTileBytes >> 4) + half * (4 * 2048 >> 4));
        const uint32_t d = tmem_base + C::kColO + tile * D;
        const uint32_t a = tmem_base + p_col + half * 32;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_ts(d, a + kk * 8, b0 + (kk * 2048 >> 4), idesc_pv, (acc || kk > 0 || half > 0) ? 1u : 0u);
      };
      auto stage_of = [&](int it) { return it % C::kStages; };
      auto parity_of = [&](int it) { return static_cast<uint32_t>((it / C::kStages) & 1); };
      auto wait_kv = [&](int it, int code) {
        return wait_or_abort(&kv_full[stage_of(it)], parity_of(it), p.status, code);
      };
      // both halves of P_tile(j), then PV_tile(j)
      auto pv_when_ready = [&](int tile, int j, int stage) {
        if (!wait_or_abort(&p_full[tile * 2], j & 1, p.status, 24 + tile)) return false;
        DTB_STAMP(2, j, 3 + 2 * tile);
        tc_fence_after();
        issue_pv(tile, stage, 0, j > 0, C::kColP + tile * C::kStrideP);
        if (!wait_or_abort(&p_full[tile * 2 + 1], j & 1, p.status, 26 + tile)) return false;
        tc_fence_after();
        issue_pv(tile, stage, 1, true, C::kColP + tile * C::kStrideP);
        return true;
      };

      bool ok = wait_or_abort(q_full, 0, p.status, 21);
      if constexpr (C::kSplit) {
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
          DTB_STAMP(2, j, 0);
          ok = wait_kv(it_v, 23);
          if (!ok) break;
          DTB_STAMP(2, j, 1);
          for (int tile = 0; tile < 2; ++tile) {
            ok = wait_or_abort(&p_full[tile * 2 + buf], (j >> 1) & 1, p.status, 24 + tile);
            if (!ok) break;
            DTB_STAMP(2, j, 2 + 2 * tile);
            tc_fence_after();
            issue_pv(tile, stage_of(it_v), 0, j > 0, C::kColS + tile * 128 + buf * kBN);
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
            DTB_STAMP(2, j, 3 + 2 * tile);
          }
        }
      } else {
      if (ok) ok = wait_kv(k_slot(0), 22);
      if (ok) {
        tc_fence_after();
        issue_s(0, stage_of(k_slot(0)));
        mma_commit(&s_full[0]);
        issue_s(1, stage_of(k_slot(0)));
        mma_commit(&s_full[1]);
        mma_commit(&kv_empty[stage_of(k_slot(0))]);
      }
      for (int j = 0; ok && j < n_tiles; ++j) {
        const bool more = (j + 1 < n_tiles);
        const int it_v = v_slot(j), it_kn = k_slot(j + 1);
        DTB_STAMP(2, j, 0);
        if (C::kDecoupled) {
          if (more) {
            ok = wait_kv(it_kn, 25);
            for (int tile = 0; ok && tile < 2; ++tile) {
              ok = wait_or_abort(&s_free[tile], j & 1, p.status, 28 + tile);
              if (!ok) break;
              tc_fence_after();
              issue_s(tile, stage_of(it_kn));
              mma_commit(&s_full[tile]);
            }
            if (!ok) break;
            mma_commit(&kv_empty[stage_of(it_kn)]);
          }
          DTB_STAMP(2, j, 1);
          ok = wait_kv(it_v, 23);
          if (!ok) break;
          DTB_STAMP(2, j, 2);
          for (int tile = 0; ok && tile < 2; ++tile) {
            ok = pv_when_ready(tile, j, stage_of(it_v));
            if (ok) mma_commit(&pv_done[tile]);
            DTB_STAMP(2, j, 4 + 2 * tile);
          }
          if (!ok) break;
          mma_commit(&kv_empty[stage_of(it_v)]);
        } else {
          ok = wait_kv(it_v, 23);
          if (!ok) break;
          DTB_STAMP(2, j, 1);
          ok = pv_when_ready(0, j, stage_of(it_v));
          if (!ok) break;
          if (more) {
            ok = wait_kv(it_kn, 25);
            if (!ok) break;
            tc_fence_after();
            issue_s(0, stage_of(it_kn));
            mma_commit(&s_full[0]);
          }
          DTB_STAMP(2, j, 2);
          ok = pv_when_ready(1, j, stage_of(it_v));
          if (!ok) break;
          mma_commit(&kv_empty[stage_of(it_v)]);
          if (more) {
            issue_s(1, stage_of(it_kn));
            mma_commit(&s_full[1]);
            mma_commit(&kv_empty[stage_of(it_kn)]);
          }
          DTB_STAMP(2, j, 3);
        }
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
    const uint32_t s_taddr = lane_base + C::kColS + tile * 128;
    const uint32_t p_taddr = lane_base + C::kColP + tile * C::kStrideP;
    const uint32_t o_taddr = lane_base + C::kColO + tile * D;
    const float c = p.scale_log2;
    float m = -INFINITY;   // running max of raw scores (lazily updated)
    float l = 0.f;         // running sum of exp2((s - m) * c)
    bool ok = true;
    const bool stamp = (lane == 0 && (warp & 3) == 0);
    (void)stamp;

    if constexpr (C::kSplit) {
      for (int j = 0; j < n_tiles; ++j) {
        const int buf = j & 1;
        const uint32_t sb_taddr = s_taddr + buf * kBN;   // S_tile(j), then P_tile(j) over its first half
        if (stamp) DTB_STAMP(tile, j, 0);
        ok = wait_or_abort(&s_full[tile * 2 + buf], (j >> 1) & 1, p.status, 31 + tile);
        if (!ok) break;
        if (stamp) DTB_STAMP(tile, j, 1);
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
        if (stamp) DTB_STAMP(tile, j, 2);
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
        if (stamp) DTB_STAMP(tile, j, 3);
        if (C::kTurns) {
          ok = wait_or_abort(&exp_turn[tile * 4 + (warp & 3)], tile == 0 ? ((j & 1) ^ 1) : (j & 1), p.status, 35 + tile);
          if (!ok) break;
        }
        if (stamp) DTB_STAMP(tile, j, 4);
        const float nmc = -m * c;
        float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
        uint32_t pk[kBN / 2];
#pragma unroll
        for (int g = 0; g < kBN / 8; ++g) {
#pragma unroll
          for (int pr = 0; pr < 4; ++pr) {
            const int i = g * 8 + pr * 2;
            const float x0 = fmaf(__uint_as_float(sr[i]), c, nmc);
            const float x1 = fmaf(__uint_as_float(sr[i + 1]), c, nmc);
            float p0, p1;
            if (pr >= 4 - C::kEmuPairs) {
              exp2_poly_pair(x0, x1, p0, p1);
            } else {
              p0 = ex2(x0);
              p1 = ex2(x1);
            }
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
        if (stamp) DTB_STAMP(tile, j, 5);
        tmem_st32(sb_taddr, pk);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&p_full[tile * 2 + buf]);
        if (stamp) DTB_STAMP(tile, j, 6);
        // Handing the turn over any earlier (after the exp loop, or part-way through it) was measured
        // 10 % slower: the two groups then drift into phase and exponentiate side by side.
        if (C::kTurns) mbar_arrive(&exp_turn[(tile ^ 1) * 4 + (warp & 3)]);
        l += (sum0 + sum1) + (sum2 + sum3);
      }
    } else {
    for (int j = 0; j < n_tiles; ++j) {
      if (stamp) DTB_STAMP(tile, j, 0);
      ok = wait_or_abort(&s_full[tile], j & 1, p.status, 31 + tile);
      if (!ok) break;
      if (stamp) DTB_STAMP(tile, j, 1);
      tc_fence_after();
      uint32_t sr[kBN];
      const bool tail = (j == n_tiles - 1) && (k_len & (kBN - 1)) != 0;
      const int valid = tail ? k_len - j * kBN : kBN;
      tmem_ld32(s_taddr, sr);
      tmem_ld32(s_taddr + 32, sr + 32);
      tmem_wait_ld();
      // the second half of the row lands while the first half is reduced
      tmem_ld32(s_taddr + 64, sr + 64);
      tmem_ld32(s_taddr + 96, sr + 96);
      if (tail) {
#pragma unroll
        for (int i = 0; i < kBN / 2; ++i)
          if (i >= valid) sr[i] = 0xff800000u;   // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < kBN / 2; i += 8) {
        mx0 = max3(mx0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
        mx1 = max3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
        mx2 = max3(mx2, __uint_as_float(sr[i + 4]), __uint_as_float(sr[i + 5]));
        mx3 = max3(mx3, __uint_as_float(sr[i + 6]), __uint_as_float(sr[i + 7]));
      }
      tmem_wait_ld();
      if (C::kDecoupled) {
        // S_tile(j) now lives in registers: the tensor pipe may overwrite it with S_tile(j+1)
        tc_fence_before();
        mbar_arrive(&s_free[tile]);
      }
      if (tail) {
#pragma unroll
        for (int i = kBN / 2; i < kBN; ++i)
          if (i >= valid) sr[i] = 0xff800000u;
      }
#pragma unroll
      for (int i = kBN / 2; i < kBN; i += 8) {
        mx0 = max3(mx0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
        mx1 = max3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
        mx2 = max3(mx2, __uint_as_float(sr[i + 4]), __uint_as_float(sr[i + 5]));
        mx3 = max3(mx3, __uint_as_float(sr[i + 6]), __uint_as_float(sr[i + 7]));
      }
      if (stamp) DTB_STAMP(tile, j, 2);
      const float m_new = fmaxf(max3(m, mx0, mx1), fmaxf(mx2, mx3));
      if (C::kDecoupled && j > 0) {
        // PV_tile(j-1) must have drained before its P columns are rewritten or O is rescaled.  (In the
        // coupled order the commit behind s_full(j) already covers it.)
        ok = wait_or_abort(&pv_done[tile], (j - 1) & 1, p.status, 33 + tile);
        if (!ok) break;
        tc_fence_after();
      }
      if (j == 0) {
        m = m_new;
      } else {
        const bool grow = (m_new - m) * c > kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
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
      if (stamp) DTB_STAMP(tile, j, 3);
      // p = 2^(s*c - m*c): the ex2 unit (16 results per clock per SM) against 4*D tensor FLOPs per
      // score; kEmuPairs of every four pairs go through the FMA/ALU pipes instead.
      if (C::kTurns) {
        // Warp w of group 0 and warp w of group 1 sit on the same scheduler and feed the same ex2
        // unit.  They take turns in the exp phase (0, 1, 0, 1, ...): side by side each phase would
        // take twice as long and the unit would idle while both warps load and reduce their next
        // rows.  Group 0's first turn is free (parity trick).
        ok = wait_or_abort(&exp_turn[tile * 4 + (warp & 3)], tile == 0 ? ((j & 1) ^ 1) : (j & 1), p.status, 35 + tile);
        if (!ok) break;
      }
      const float nmc = -m * c;
      float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
      uint32_t pk[kBN / 2];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int g = half * 8; g < half * 8 + 8; ++g) {
#pragma unroll
          for (int pr = 0; pr < 4; ++pr) {
            const int i = g * 8 + pr * 2;
            const float x0 = fmaf(__uint_as_float(sr[i]), c, nmc);
            const float x1 = fmaf(__uint_as_float(sr[i + 1]), c, nmc);
            float p0, p1;
            if (pr >= 4 - C::kEmuPairs) {
              exp2_poly_pair(x0, x1, p0, p1);
            } else {
              p0 = ex2(x0);
              p1 = ex2(x1);
            }
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
        tmem_st32(p_taddr + half * 32, pk + half * 32);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&p_full[tile * 2 + half]);
        if (stamp) DTB_STAMP(tile, j, 4 + half);
      }
      if (C::kTurns) mbar_arrive(&exp_turn[(tile ^ 1) * 4 + (warp & 3)]);
      l += (sum0 + sum1) + (sum2 + sum3);
    }
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
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64) {
    std::lock_guard<std::mutex> lk(mu);
    if (!configured[dev]) {
      cudaError_t e = cudaFuncSetAttribute(flash_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
      if (e != cudaSuccess) return e;
      configured[dev] = true;
    }
  }
  dim3 grid((p.seqlen_q + kQT * kBM - 1) / (kQT * kBM), p.num_heads, p.nseg);
  flash_fwd_kernel<D><<<grid, kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, p);
  return cudaGetLastError();
}

int flash_kv_box_rows(int head_dim) { return head_dim == 128 ? Cfg<128>::kBN : Cfg<64>::kBN; }

#ifdef DTB_FLASH_TIMING
cudaError_t read_flash_timing(long long* host, int n) {
  return cudaMemcpyFromSymbol(host, g_flash_timing, sizeof(long long) * n);
}
#endif

template cudaError_t launch_flash<64>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const FlashParams&, cudaStream_t);
template cudaError_t launch_flash<128>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const FlashParams&, cudaStream_t);

}  // namespace dtb
