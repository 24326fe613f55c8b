// Partial-attention forward, two threads per query row: the kernel used at head dimension 64, where one
// ex2 per score against 4 x 64 tensor FLOPs makes the softmax side, not the tensor pipe, the bound.
//
// CTA = 256 query rows of one (segment, head): two 128-row Q tiles share the tensor core.  Warp roles
// (640 threads, five warpgroups):
//   warps 0-15  softmax: TWO threads per query row.  Warp w serves rows 32 (w % 4) .. + 32 of Q tile
//               (w / 4) % 2 and the key half w / 8 of every 64-key tile (32 scores per thread and tile).
//   warp  16    TMA producer: Q tiles once, then K_j, V_j tiles (64 keys each) through a shared-memory ring
//   warp  17    MMA issuer (one elected thread): S_i = Q_i K_j^T and O_i += P_i V_j via tcgen05.mma
//   warps 18-19 no role; they complete the fifth warpgroup so that it can hand registers over
// Four softmax warps per scheduler instead of two: the tensor-memory round trips, the barrier waits and the
// ex2 latency of one warp are covered by the other three, which a thread-per-row layout cannot do.
//
// Tensor memory (512 columns x 128 lanes of fp32): per Q tile i two S buffers of 64 columns at
// [128 i, 128 i + 64) and [128 i + 64, 128 i + 128), and the O accumulator at [256 + D i, 256 + D i + D).
// S_i(j) sits in buffer j & 1.  Each thread overwrites the first 16 columns of ITS OWN 32-column half with
// its bf16 probabilities, so P_i(j) lies in two pieces (keys 0-31 at column 0, keys 32-63 at column 32) and
// neither thread touches scores the other still has to read.  S_i(j+2) is issued right behind PV_i(j):
//     S0(0) S1(0) S0(1) S1(1) | PV0(j) S0(j+2) PV1(j) S1(j+2) | ...
//
// At D = 64 tensor memory has room for three S buffers per tile; S_i(j+3) then follows PV_i(j), the tensor
// pipe runs two key tiles ahead of the softmax threads, and the reference lags three tiles instead of two.
//
// A thread's 32 scores come from tensor memory in two loads of 16.  The second is in flight while the
// first 16 are exponentiated, and the first 16 of the NEXT tile are requested as soon as their registers
// are free (if that tile is already complete), so the round trip of a tensor-memory load is rarely waited for.
//
// The two threads of a row must exponentiate against the same reference value m.  They agree on it
// without waiting for each other: every thread publishes the maximum of its half of tile j in shared
// memory, and the reference used for tile j is the running maximum over the tiles up to j - 2 of both
// halves (tile 0: one real exchange; "2" is the number of S buffers).  A value that old is certain to be
// visible: the partner wrote it before handing over P(j-2), which the issuer needs before it can issue S(j).  Probabilities may then
// exceed 1 by what the last two tiles add to the maximum; fp32 / bf16 have the range for that, and O and
// the row sums are rescaled (each thread its half of the O columns) when the reference grows by more
// than 2^8.  The final normalisation undoes all of it.
#include "flash_common.cuh"

#include <mutex>

namespace dtb {

namespace {

using namespace flash;

// Packed two-wide fp32 arithmetic (fma.rn.f32x2, add.rn.f32x2) for the score scaling and the row sums:
// fewer issue slots per score with four softmax warps per scheduler.
#ifndef DTB_F32X2
#define DTB_F32X2 1
#endif

constexpr int kThreads = 640;
constexpr int kRegsSoftmax = 104;   // the kernel starts at 96 per thread: 4 x 128 x 8 registers taken ...
constexpr int kRegsOther = 64;      // ... are the 128 x 32 the fifth warpgroup gives up
constexpr int kTmaWarp = 16;
constexpr int kMmaWarp = 17;
constexpr int kHalf = kBN / 2;      // scores per thread and key tile
constexpr int kChunk = kHalf / 2;   // ... which arrive from tensor memory in two loads of 16
constexpr int kRing = 8;            // key tiles whose half-row maxima are kept in shared memory

template <int D>
struct Cfg {
  static constexpr int kSlabs = D / 64;
  static constexpr int kTileBytes = kBM * D * 2;          // one Q tile
  static constexpr int kKvTileBytes = kBN * D * 2;        // one K or V tile
  static constexpr int kStages = (D == 128) ? 8 : 12;
  // S buffers per Q tile (64 columns each): as many as tensor memory has room for beside the O accumulators
#ifdef DTB_SBUFS
  static constexpr int kSBufs = DTB_SBUFS;
#else
  static constexpr int kSBufs = (512 - kQT * D) / (kQT * kBN) >= 3 ? 3 : 2;
#endif
  // barriers: q_full, kv_full[S], kv_empty[S], s_full[2 L], p_full[2 L], pv_done[2 L], o_final, pair[8]
  static constexpr int kBars = 1 + 2 * kStages + 6 * kSBufs + 1 + 8;
  // half-row maxima of the last kRing key tiles [kRing][tile][row][half], and the row sums exchanged at the end
  static constexpr int kExchangeBytes = (kRing + 1) * kQT * kBM * 2 * 4;
  static constexpr int kSmemBytes = 1024 + kQT * kTileBytes + kStages * kKvTileBytes + kExchangeBytes + kBars * 8 + 16;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kColS = 0;                        // + tile * kTileS + buffer * 64
  static constexpr uint32_t kTileS = kSBufs * kBN;            // S columns of one Q tile
  static constexpr uint32_t kColO = kQT * kSBufs * kBN;       // + tile * D
  static_assert(kColO + kQT * D <= 512, "tensor memory");
};

#ifdef DTB_FLASH_TIMING
// softmax phases: 0 top of step, 1 S ready and first load issued, 2 first 16 scores in registers, 3 exp done,
//                 4 P handed over;
// issuer phases:  0 top of step, 1 V ready, 2 P0 ready, 3 PV0 + S0(j+L) issued, 4 P1 ready, 5 PV1 + S1(j+L) issued.
__device__ long long g_timing_pair[3 * 48 * 8];
#endif
#define STAMP(role, j, phase) DTB_STAMP(g_timing_pair, role, j, phase)
#define STAMP_IF(cond, role, j, phase) do { if (cond) STAMP(role, j, phase); } while (0)

// Row sums: four independent accumulators (two packed pairs when DTB_F32X2).
struct RowSum {
#if DTB_F32X2
  uint64_t a, b;
  __device__ __forceinline__ void clear() { a = b = pack2(0.f, 0.f); }
  __device__ __forceinline__ void add(int slot, float p0, float p1) {
    if (slot & 1) b = add2(b, pack2(p0, p1)); else a = add2(a, pack2(p0, p1));
  }
  __device__ __forceinline__ float total() const {
    float a0, a1, b0, b1;
    unpack2(a, a0, a1);
    unpack2(b, b0, b1);
    return (a0 + a1) + (b0 + b1);
  }
#else
  float s0, s1, s2, s3;
  __device__ __forceinline__ void clear() { s0 = s1 = s2 = s3 = 0.f; }
  __device__ __forceinline__ void add(int slot, float p0, float p1) {
    if (slot & 1) { s2 += p0; s3 += p1; } else { s0 += p0; s1 += p1; }
  }
  __device__ __forceinline__ float total() const { return (s0 + s1) + (s2 + s3); }
#endif
};

// p = 2^(s*c - m*c) for the 8 elements [8 g, 8 g + 8) of a 16-score chunk; bf16 pairs into pk[4 og .. 4 og + 4).
__device__ __forceinline__ void exp_group(const uint32_t (&row)[kChunk], uint32_t (&pk)[kHalf / 2], int g, int og, float c,
                                          float nmc, RowSum& sum) {
#pragma unroll
  for (int pr = 0; pr < 4; ++pr) {
    const int i = g * 8 + pr * 2;
#if DTB_F32X2
    float x0, x1;
    unpack2(fma2(pack2(__uint_as_float(row[i]), __uint_as_float(row[i + 1])), pack2(c, c), pack2(nmc, nmc)), x0, x1);
#else
    const float x0 = fmaf(__uint_as_float(row[i]), c, nmc);
    const float x1 = fmaf(__uint_as_float(row[i + 1]), c, nmc);
#endif
    const float p0 = ex2(x0), p1 = ex2(x1);
    sum.add(pr, p0, p1);
    pk[og * 4 + pr] = pack_bf16x2(p0, p1);
  }
}

}  // namespace

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
flash_fwd_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const FlashParams p) {
  using C = Cfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem;
  uint8_t* s_kv = smem + kQT * C::kTileBytes;
  float* s_hmax = reinterpret_cast<float*>(s_kv + C::kStages * C::kKvTileBytes);   // [kRing][tile][row][half]
  float* s_lsum = s_hmax + kRing * kQT * kBM * 2;                                  // [tile][row][half]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_lsum + kQT * kBM * 2);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + C::kStages;
  constexpr int L = C::kSBufs;
  uint64_t* s_full = kv_empty + C::kStages;   // [tile*L + buffer]: S_tile(j) is in tensor memory
  uint64_t* p_full = s_full + 2 * L;          // [tile*L + buffer]: P_tile(j) written (one arrival per softmax warp: 8)
  uint64_t* pv_done = p_full + 2 * L;         // [tile*L + buffer]: PV_tile(j) has completed
  uint64_t* o_final = pv_done + 2 * L;
  uint64_t* pair = o_final + 1;               // [tile*4 + quarter]: the two warps that share 32 rows meet here
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

  // Position of K_j / V_j in the order the ring carries them (L = S buffers per tile):
  //   K_0 .. K_{L-1} | V_0 K_L | V_1 K_{L+1} | ... | V_{n-L-1} K_{n-1} | V_{n-L} .. V_{n-1}
  // (K_{j+L} follows V_j, as S(j+L) follows PV(j) on the pipe).
  const int n_lead = n_tiles < L ? n_tiles : L;
  auto v_slot = [&](int j) { const int k_before = j < n_tiles - L ? j : (n_tiles - L > 0 ? n_tiles - L : 0); return n_lead + j + k_before; };
  auto k_slot = [&](int j) { return j < L ? j : v_slot(j - L) + 1; };

  // ------------------------------------------------------------------ set-up
  if (threadIdx.x == kTmaWarp * 32) {
    mbar_init(q_full, 1);
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 2 * L; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 8);
    }
    for (int i = 0; i < 2 * L; ++i) mbar_init(&pv_done[i], 1);
    for (int i = 0; i < 8; ++i) mbar_init(&pair[i], 2);
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

  if (warp >= 16) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
  if (aborted || warp > kMmaWarp) {
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
      int it = 0;
      bool live = true;
      auto load_tile = [&](bool is_v, int j) {
        const int stage = it % C::kStages;
        const int round = it / C::kStages;
        ++it;
        if (round > 0 && !wait_or_abort(&kv_empty[stage], (round - 1) & 1, p.status, 11)) return false;
        mbar_expect_tx(&kv_full[stage], C::kKvTileBytes);
        const CUtensorMap* tm = is_v ? &tm_v : &tm_k;
        const int row = k_begin + j * kBN;
        for (int s = 0; s < C::kSlabs; ++s)
          tma_load_2d(s_kv + stage * C::kKvTileBytes + s * kKvSlabBytes, tm, &kv_full[stage], head * D + s * 64, row);
        return true;
      };
      for (int j = 0; live && j < n_lead; ++j) live = load_tile(false, j);
      for (int j = 0; live && j < n_tiles; ++j) {
        live = load_tile(true, j);
        if (live && j + L < n_tiles) live = load_tile(false, j + L);
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
        const uint32_t d = tmem_base + C::kColS + tile * C::kTileS + s_col;
#pragma unroll
        for (int k16 = 0; k16 < D / 16; ++k16) {
          const uint32_t in_slab = (k16 & 3) * 32;
          mma_ss(d, a0 + (((k16 >> 2) * kSlabBytes + in_slab) >> 4), b0 + (((k16 >> 2) * kKvSlabBytes + in_slab) >> 4),
                 idesc_qk, k16 > 0);
        }
      };
      // O_tile (+)= P_tile V: four K=16 steps over the 64 keys.  P (bf16 pairs) starts at tensor-memory column
      // p_col: keys 0-31 in columns [0, 16), keys 32-63 in columns [32, 48) (each softmax thread writes over
      // the start of its own half of the S buffer).
      auto issue_pv = [&](int tile, int stage, bool acc, uint32_t p_col) {
        const uint64_t b0 = v_desc + static_cast<uint32_t>(stage * (C::kKvTileBytes >> 4));
        const uint32_t d = tmem_base + C::kColO + tile * D;
        const uint32_t a = tmem_base + p_col;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_ts(d, a + (kk >> 1) * kHalf + (kk & 1) * 8, b0 + (kk * 2048 >> 4), idesc_pv, (acc || kk > 0) ? 1u : 0u);
      };
      auto stage_of = [&](int it) { return it % C::kStages; };
      auto parity_of = [&](int it) { return static_cast<uint32_t>((it / C::kStages) & 1); };
      auto wait_kv = [&](int it, int code) {
        return wait_or_abort(&kv_full[stage_of(it)], parity_of(it), p.status, code);
      };

      bool ok = wait_or_abort(q_full, 0, p.status, 21);
      // S(0) .. S(L-1) of both Q tiles fill the buffers; from then on S(j+L) follows PV(j).
      for (int j = 0; ok && j < n_lead; ++j) {
        ok = wait_kv(k_slot(j), 22);
        if (!ok) break;
        tc_fence_after();
        for (int tile = 0; tile < 2; ++tile) {
          issue_s(tile, stage_of(k_slot(j)), j * kBN);
          mma_commit(&s_full[tile * L + j]);
        }
        mma_commit(&kv_empty[stage_of(k_slot(j))]);
      }
      int buf = 0;
      uint32_t use = 0;           // how often this buffer has been used before: parity of its barriers
      for (int j = 0; ok && j < n_tiles; ++j) {
        const bool more = (j + L < n_tiles);
        const int it_v = v_slot(j), it_kn = k_slot(j + L);
        STAMP(2, j, 0);
        ok = wait_kv(it_v, 23);
        if (!ok) break;
        STAMP(2, j, 1);
        for (int tile = 0; tile < 2; ++tile) {
          ok = wait_or_abort(&p_full[tile * L + buf], use & 1, p.status, 24 + tile);
          if (!ok) break;
          STAMP(2, j, 2 + 2 * tile);
          tc_fence_after();
          issue_pv(tile, stage_of(it_v), j > 0, C::kColS + tile * C::kTileS + buf * kBN);
          mma_commit(&pv_done[tile * L + buf]);
          if (tile == 1) mma_commit(&kv_empty[stage_of(it_v)]);
          if (more) {
            if (tile == 0) {
              ok = wait_kv(it_kn, 25);
              if (!ok) break;
              tc_fence_after();
            }
            // overwrites P_tile(j); the pipe runs it behind PV_tile(j)
            issue_s(tile, stage_of(it_kn), buf * kBN);
            mma_commit(&s_full[tile * L + buf]);
            if (tile == 1) mma_commit(&kv_empty[stage_of(it_kn)]);
          }
          STAMP(2, j, 3 + 2 * tile);
        }
        if (++buf == L) { buf = 0; ++use; }
      }
      if (ok) mma_commit(o_final);
    }
    __syncwarp();
  }
  } else {
    // -------------------------------------------------------------- softmax + epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    const int quarter = warp & 3;
    const int tile = (warp >> 2) & 1;
    const int half = warp >> 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_taddr = lane_base + C::kColS + tile * C::kTileS + half * kHalf;   // + buffer * 64: this thread's scores
    const uint32_t o_taddr = lane_base + C::kColO + tile * D + half * (D / 2);         // this thread's half of the O row
    float* my_hmax = s_hmax + (tile * kBM + row) * 2;        // + slot * (kQT * kBM * 2); [0] = half 0, [1] = half 1
    constexpr int kSlotPitch = kQT * kBM * 2;
    uint64_t* pair_bar = &pair[tile * 4 + quarter];
    const float c = p.scale_log2;
    const bool stamp = (lane == 0 && quarter == 0 && half == 0);
    (void)stamp;
    float m = -INFINITY;   // reference value the row's probabilities are taken against (raw-score units)
    float l = 0.f;         // this thread's part of the row sum
    bool ok = !aborted;
    const bool ragged = (k_len & (kBN - 1)) != 0;

    // scores of the current tile: first 16 in sa, second 16 in sb
    uint32_t sa[kChunk], sb[kChunk];
    int buf = 0;
    uint32_t use = 0;               // parity of this buffer's barriers
    bool a_loaded = false;          // sa already requested for the coming tile
    for (int j = 0; ok && j < n_tiles; ++j) {
      STAMP_IF(stamp, tile, j, 0);
      const uint32_t s_addr = s_taddr + buf * kBN;
      if (!a_loaded) {
        ok = wait_or_abort(&s_full[tile * L + buf], use & 1, p.status, 31 + tile);
        if (!ok) break;
        tc_fence_after();
        tmem_ld16(s_addr, sa);
      }
      STAMP_IF(stamp, tile, j, 1);
      if (j >= L) {
        // reference for this tile: what both halves had seen L tiles ago
        const volatile float* h = my_hmax + ((j - L) & (kRing - 1)) * kSlotPitch;
        const float m_new = max3(m, h[0], h[1]);
        const bool grow = (m_new - m) * c > kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
          // O is rescaled in place, each thread its half of the columns: PV(j-1) must have drained; PV(j)
          // is not issued before all eight warps of the tile have handed over P(j).  (One barrier per
          // buffer: with a single one, a laggard could mistake the completion of PV(j-3) for that of PV(j-1).)
          const int pbuf = (buf == 0) ? L - 1 : buf - 1;
          const uint32_t puse = (buf == 0) ? use - 1 : use;
          ok = wait_or_abort(&pv_done[tile * L + pbuf], puse & 1, p.status, 33 + tile);
          if (!ok) break;
          tc_fence_after();
          tmem_wait_ld();          // sa first: the loads below reuse the wait
          const float f = ex2((m - m_new) * c);
#pragma unroll
          for (int q = 0; q < D / 32; ++q) {
            uint32_t orow[kChunk];
            tmem_ld16(o_taddr + q * kChunk, orow);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < kChunk; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * f);
            tmem_st16(o_taddr + q * kChunk, orow);
          }
          tmem_wait_st();
          l *= f;
          m = m_new;
        }
      }
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < kChunk; i += 8)
        asm volatile("" : "+r"(sa[i]), "+r"(sa[i + 1]), "+r"(sa[i + 2]), "+r"(sa[i + 3]), "+r"(sa[i + 4]), "+r"(sa[i + 5]),
                          "+r"(sa[i + 6]), "+r"(sa[i + 7]));
      tmem_ld16(s_addr + kChunk, sb);                       // in flight while sa is worked on
      const bool last_ragged = ragged && (j == n_tiles - 1);
      const int valid = last_ragged ? k_len - j * kBN - half * kHalf : kHalf;      // of this thread's 32 keys
      if (last_ragged) {
#pragma unroll
        for (int i = 0; i < kChunk; ++i)
          if (i >= valid) sa[i] = 0xff800000u;   // -inf
      }
      float mx0 = max3(__uint_as_float(sa[0]), __uint_as_float(sa[1]), __uint_as_float(sa[2]));
      float mx1 = max3(__uint_as_float(sa[3]), __uint_as_float(sa[4]), __uint_as_float(sa[5]));
      float mx2 = max3(__uint_as_float(sa[6]), __uint_as_float(sa[7]), __uint_as_float(sa[8]));
      float mx3 = max3(__uint_as_float(sa[9]), __uint_as_float(sa[10]), __uint_as_float(sa[11]));
      mx0 = max3(mx0, __uint_as_float(sa[12]), __uint_as_float(sa[13]));
      mx1 = max3(mx1, __uint_as_float(sa[14]), __uint_as_float(sa[15]));
      if (j == 0) {
        // the one real exchange: both halves of tile 0 give the starting reference (needs the whole row)
        tmem_wait_ld();
        if (last_ragged) {
#pragma unroll
          for (int i = 0; i < kChunk; ++i)
            if (i + kChunk >= valid) sb[i] = 0xff800000u;
        }
#pragma unroll
        for (int i = 0; i < kChunk; i += 4) {
          mx2 = max3(mx2, __uint_as_float(sb[i]), __uint_as_float(sb[i + 1]));
          mx3 = max3(mx3, __uint_as_float(sb[i + 2]), __uint_as_float(sb[i + 3]));
        }
        my_hmax[half] = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        __syncwarp();
        if (lane == 0) mbar_arrive(pair_bar);
        ok = wait_or_abort(pair_bar, 0, p.status, 35 + tile);
        if (!ok) break;
        const volatile float* h = my_hmax;
        m = fmaxf(h[0], h[1]);
      }
      STAMP_IF(stamp, tile, j, 2);
      const float nmc = -m * c;
      RowSum sum;
      sum.clear();
      uint32_t pk[kHalf / 2];
      exp_group(sa, pk, 0, 0, c, nmc, sum);
      exp_group(sa, pk, 1, 1, c, nmc, sum);
      tmem_wait_ld();                                        // sb
#pragma unroll
      for (int i = 0; i < kChunk; i += 8)
        asm volatile("" : "+r"(sb[i]), "+r"(sb[i + 1]), "+r"(sb[i + 2]), "+r"(sb[i + 3]), "+r"(sb[i + 4]), "+r"(sb[i + 5]),
                          "+r"(sb[i + 6]), "+r"(sb[i + 7]));
      // sa's registers are free: ask for the first 16 scores of the next tile if it is already complete
      // (never wait for it here: P(j) must not depend on S(j+1))
      a_loaded = false;
      {
        const int nbuf = (buf + 1 == L) ? 0 : buf + 1;
        const uint32_t nuse = (buf + 1 == L) ? use + 1 : use;
        if (j + 1 < n_tiles && __all_sync(0xffffffffu, mbar_try_wait(&s_full[tile * L + nbuf], nuse & 1))) {
          tc_fence_after();
          tmem_ld16(s_taddr + nbuf * kBN, sa);
          a_loaded = true;
        }
      }
      if (j > 0) {
        if (last_ragged) {
#pragma unroll
          for (int i = 0; i < kChunk; ++i)
            if (i + kChunk >= valid) sb[i] = 0xff800000u;
        }
#pragma unroll
        for (int i = 0; i < kChunk; i += 4) {
          mx2 = max3(mx2, __uint_as_float(sb[i]), __uint_as_float(sb[i + 1]));
          mx3 = max3(mx3, __uint_as_float(sb[i + 2]), __uint_as_float(sb[i + 3]));
        }
        my_hmax[(j & (kRing - 1)) * kSlotPitch + half] = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      }
      exp_group(sb, pk, 0, 2, c, nmc, sum);
      exp_group(sb, pk, 1, 3, c, nmc, sum);
      STAMP_IF(stamp, tile, j, 3);
      // P(j) over the start of this thread's own half of the S buffer, then one arrival per warp
      tmem_st16(s_addr, pk);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[tile * L + buf]);
      STAMP_IF(stamp, tile, j, 4);
      l += sum.total();
      if (++buf == L) { buf = 0; ++use; }
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
      int64_t li = 0;
      float lse_old = -INFINITY;
      if (valid) {
        li = lse_index(p, seg, head, q_pos, tok);
        if (p.accumulate) lse_old = p.lse[li];        // read by both halves before either writes the new value
      }
      // the row sum is the two halves' sums (both taken against the same reference m)
      s_lsum[(tile * kBM + row) * 2 + half] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(pair_bar);
      ok = wait_or_abort(pair_bar, 1, p.status, 37 + tile);
      if (ok) {
        const volatile float* ls = s_lsum + (tile * kBM + row) * 2;
        const float l_row = ls[0] + ls[1];
        const float lse_new = (m * c + log2f(l_row)) * kLn2;
        float w_new, w_old, lse_out;
        merge_weights(p.accumulate != 0, lse_old, lse_new, l_row, w_new, w_old, lse_out);
        if (valid && half == 0) p.lse[li] = lse_out;
#pragma unroll
        for (int q = 0; q < D / 64; ++q) {
          uint32_t orow[32];
          tmem_ld32(o_taddr + q * 32, orow);
          tmem_wait_ld();
          if (valid) store_row_chunk32(p, tok, static_cast<int64_t>(head) * D + half * (D / 2) + q * 32, orow, w_new, w_old);
        }
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
cudaError_t launch_flash_pair(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FlashParams& p,
                              cudaStream_t stream) {
  using C = Cfg<D>;
  static bool configured[64] = {};
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64) {
    std::lock_guard<std::mutex> lk(mu);
    if (!configured[dev]) {
      cudaError_t e = cudaFuncSetAttribute(flash_fwd_pair_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
      if (e != cudaSuccess) return e;
      configured[dev] = true;
    }
  }
  dim3 grid((p.seqlen_q + kQT * kBM - 1) / (kQT * kBM), p.num_heads, p.nseg);
  return launch_attention_kernel(flash_fwd_pair_kernel<D>, grid, kThreads, C::kSmemBytes, stream, p.overlap_previous != 0, tq, tk, tv, p);
}

#ifdef DTB_FLASH_TIMING
cudaError_t read_flash_timing_pair(long long* host, int n) {
  return cudaMemcpyFromSymbol(host, g_timing_pair, sizeof(long long) * n);
}
#endif

template cudaError_t launch_flash_pair<64>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const FlashParams&, cudaStream_t);
template cudaError_t launch_flash_pair<128>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const FlashParams&, cudaStream_t);

}  // namespace dtb
