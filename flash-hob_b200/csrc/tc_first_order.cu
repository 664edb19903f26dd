// Forward and first backward of attention on the tensor cores (sm_100a): the producers of the
// tensors the double-backward operator consumes (O, L) and the first-order half of a
// twice-differentiable attention function (dQ, dK, dV).  Role of the reference's forward kernel
// and of its dense backward (fhog/triton_flash.py:12-133, :190-220), at O(N) memory.
//
// Same building blocks as the double-backward kernels: TMA tile loads, tcgen05.mma with fp32
// accumulators in TMEM, elementwise math on tcgen05.ld'ed registers, 16-bit tiles written back
// to TMEM as the A operand of the output products.  The pipeline is simpler, because TMEM has
// room for two score stages in every mode: the issuing warp runs one tile ahead,
//     scores(t+1) -> stage (t+1)%2 | wait for the 16-bit tiles of t | outputs(t) from stage t%2,
// and MMAs execute in issue order, so stage t%2 is only overwritten by scores(t+2) after
// outputs(t) have read it.
//
//   ONE  (queries stationary, 128 keys per tile): single-sweep forward.  Online softmax against a
//        reference maximum that follows the running row maximum lazily (only when it has grown by
//        more than 8 in the log2 domain); on those occasions the threads rescale their part of O
//        in TMEM, which is idle between two P V products.  Writes O and L.
//   LSE  (queries stationary, 128 keys per tile): S = Q K^T; online log-sum-exp -> L (fp32) only,
//        for callers that need the logsumexp but not O (role of the reference's produce_L)
//   BQ   (queries stationary,  64 keys per tile): dS = P (dP - D), dP = dO V^T;  dQ += dS K
//   BK   (keys stationary,  64 queries per tile): transposed tiles;  dV += P^T dO, dK += dS^T Q
// The backward follows jax_refs/flash_impl.py:124-173 with P = exp(S - L) and D = rowsum(dO * O).
#include <type_traits>

#include "tc_common.cuh"

namespace fhob {
namespace {

enum { FO_LSE = 0, FO_BQ = 2, FO_BK = 3, FO_ONE = 4 };
constexpr int FO_TAIL = 3072;  // barriers, TMEM base, abort flag, (max, sum) exchange

// Two head dims: the first stationary and the first streamed tile of every mode are q/k-side
// tensors (DQK columns), the second ones v-side tensors (DV columns):
//   ONE: Q | K, V     LSE: Q | K     BQ: Q, dO | K, V     BK: K, V | Q, dO
template <int MODE, int DQK, int DV>
struct FoCfg {
  static constexpr bool kQStat = MODE != FO_BK;
  static constexpr bool kForward = MODE == FO_LSE || MODE == FO_ONE;
  static constexpr int BN = kForward ? 128 : 64;
  static constexpr int NSTAT = kForward ? 1 : 2;
  static constexpr int NSTRM = MODE == FO_LSE ? 1 : 2;
  static constexpr int NACC = kForward ? 1 : 2;          // score tiles of a stage: S | S | S, dP | S^T, dP^T
  static constexpr int NOUT = MODE == FO_LSE ? 0 : (MODE == FO_BK ? 2 : 1);
  __host__ __device__ static constexpr int tile_d(int i) { return i == 0 ? DQK : DV; }
  static constexpr int OUT0_COLS = NOUT == 0 ? 0 : (MODE == FO_ONE ? DV : DQK);   // O | dQ | dK
  static constexpr int OUT1_COLS = NOUT == 2 ? DV : 0;                            // dV
  static constexpr int OUT_COLS = OUT0_COLS + OUT1_COLS;
  static constexpr int STAGE_COLS = NACC * BN;
  __host__ __device__ static constexpr int stat_off(int i) { return i == 0 ? 0 : stat_off(i - 1) + BM * tile_d(i - 1) * 2; }
  __host__ __device__ static constexpr int strm_off(int i) { return i == 0 ? 0 : strm_off(i - 1) + BN * tile_d(i - 1) * 2; }
  static constexpr int STAT_BYTES = stat_off(NSTAT);
  static constexpr int STRM_BYTES = strm_off(NSTRM);
  // BK: -L*log2e and -D of the streamed queries travel with the slot
  static constexpr int VEC_BYTES = MODE == FO_BK ? 2 * BN * 4 : 0;
  static constexpr int TX_BYTES = STRM_BYTES + VEC_BYTES;
  static constexpr int SLOT_BYTES = STRM_BYTES + (VEC_BYTES ? 1024 : 0);  // tiles stay 1024-byte aligned
  static constexpr int NSLOT_FIT = (SMEM_LIMIT - FO_TAIL - STAT_BYTES) / SLOT_BYTES;
  static constexpr int NSLOT = NSLOT_FIT > 4 ? 4 : NSLOT_FIT;
  static constexpr int SMEM_BYTES = STAT_BYTES + NSLOT * SLOT_BYTES + FO_TAIL;
  static_assert(OUT_COLS + 2 * STAGE_COLS <= TMEM_COLS, "TMEM budget");
  static_assert(NSLOT >= 2, "need two streamed slots");
  static_assert((DQK == 64 || DQK == 128) && (DV == 64 || DV == 128), "head dims");
};

struct FoParams {
  CUtensorMap stat[2];
  CUtensorMap strm[2];
  const float* nlc;   // BQ, BK: -L*log2(e) per query
  const float* k1;    // BQ, BK: -D per query
  float* lse_out;     // LSE
  uint16_t* out0;     // ONE: O;  BQ: dQ;  BK: dK
  uint16_t* out1;     // BK: dV
  int* status;
  int n_q, n_k, causal, window, tiles_per_head;
  int heads;            // heads per batch entry of the input tensor maps (4-D: columns, rows, head, batch)
  int d_out0, d_out1;   // columns of the results in memory (<= the tile widths; see fo_launch)
  float scale;
};

struct FoBars {
  uint64_t stat_full;
  uint64_t strm_full[4];
  uint64_t strm_free[4];
  uint64_t s_full[2];   // scores of a stage finished
  uint64_t s_free[2];   // LSE: stage read by the elementwise warps
  uint64_t p_full[2];   // 16-bit tiles of a stage written
  uint64_t out_full;
  uint64_t o_done;      // ONE: the P V product of a tile has finished (O may be rescaled)
  uint64_t pair[4];     // ONE: the two warps that share 32 rows have both published their maximum
  uint64_t go[2];       // BQ, BK: the outputs that read stage [i] have been issued (its dP columns may be reused)
  uint64_t teardown[2];
  uint32_t tmem_base;
  int abort_flag;
  float red[2][2][BM];  // exchange of maxima / sums between the two column halves: [tile parity][half][row]
};
static_assert(sizeof(FoBars) <= FO_TAIL, "tail");

// fp32 problems (SPLIT): the split-operand scheme of the double-backward kernels (tc_kernels.cu):
// every fp32 operand as bf16 hi + lo, rows [hi(64) | lo(64)] = the two boxes of a 128-wide tile,
// three products per contraction, 16-bit tiles handed back as hi and lo halves, the two halves
// of an output accumulator added in the epilogue.  Head dims 64, instantiated as 128/128.
__device__ __forceinline__ void fo_split_pack(float x, float y, uint32_t& hi, uint32_t& lo) {
  hi = pack_bf16(x, y);
  lo = pack_bf16(x - __uint_as_float(hi << 16), y - __uint_as_float(hi & 0xffff0000u));
}

template <int A_BOX, int B_BOX>
__device__ __forceinline__ void fo_gemm_ss_split(bool leader, uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                                 uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int term = 0; term < 3; ++term) {   // (hi, hi), (hi, lo), (lo, hi)
    const int ab = term == 2 ? 1 : 0, bb = term == 1 ? 1 : 0;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
      umma_ss_split(d_tmem, a_lo + ((ab * A_BOX + ks * 32) >> 4), b_lo + ((bb * B_BOX + ks * 32) >> 4), kDescHi, idesc,
                    (accumulate || term > 0 || ks > 0) ? 1u : 0u, leader);
  }
}

template <int MODE, int DQK, int DV, bool F16, bool SPLIT = false>
__global__ void __launch_bounds__(NTHREADS, 1) fo_kernel(const __grid_constant__ FoParams p) {
  using C = FoCfg<MODE, DQK, DV>;
  static_assert(!SPLIT || (DQK == 128 && DV == 128 && !F16), "split fp32 operands are [hi(64) | lo(64)] bf16 rows");
  constexpr bool kQStat = C::kQStat;
  constexpr int BN = C::BN;
  constexpr int CPT = BN / 2;  // fp32 columns of a score tile per elementwise thread
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* stat_tiles = smem;
  uint8_t* strm_tiles = smem + C::STAT_BYTES;
  FoBars* bars = reinterpret_cast<FoBars*>(strm_tiles + C::NSLOT * C::SLOT_BYTES);
  int* status = p.status;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x / p.tiles_per_head;
  const int tile_in_head = blockIdx.x - head * p.tiles_per_head;
  const int tile = kQStat ? p.tiles_per_head - 1 - tile_in_head : tile_in_head;  // causal: longest first
  const int m0 = tile * BM;
  const int n_stat = kQStat ? p.n_q : p.n_k;
  const int n_strm = kQStat ? p.n_k : p.n_q;
  const int off = p.n_k - p.n_q;
  int t_begin, t_end;
  visible_tiles(kQStat, m0, BM, BN, n_strm, off, p.causal, p.window, t_begin, t_end);
  const int n_iter = t_end - t_begin;

  if (threadIdx.x == 0) {
    if (smem_u32(smem) & 1023u) atomicOr(status, FHOB_ERR_SMEM_ALIGN);
    mbar_init(&bars->stat_full, 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&bars->strm_full[i], 1);
      mbar_init(&bars->strm_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->s_full[i], C::NACC);  // one commit per issuing warp
      mbar_init(&bars->s_free[i], EW_THREADS);
      mbar_init(&bars->p_full[i], EW_THREADS);
      mbar_init(&bars->go[i], 1);
      mbar_init(&bars->teardown[i], 1);
    }
    mbar_init(&bars->out_full, 1);
    mbar_init(&bars->o_done, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&bars->pair[i], 64);
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == TMA_WARP && lane == 0) {
    for (int i = 0; i < C::NSTAT; ++i) prefetch_tensormap(&p.stat[i]);
    for (int i = 0; i < C::NSTRM; ++i) prefetch_tensormap(&p.strm[i]);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // the CTA allocates all 512 columns, so the allocation starts at column 0 (checked)
  constexpr uint32_t tmem_base = 0;
  if (threadIdx.x == 0 && *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base) != 0)
    atomicOr(status, FHOB_ERR_TMEM_BASE);

  if (warp == TMA_WARP) {
    // ================================================= TMA producer
    if (lane == 0 && n_iter > 0) {
      const int head_b = head / p.heads, head_h = head - head_b * p.heads;   // batch entry and head within it
      mbar_arrive_expect_tx(&bars->stat_full, C::STAT_BYTES);
#pragma unroll
      for (int i = 0; i < C::NSTAT; ++i)
        for (int bx = 0; bx < C::tile_d(i) / 64; ++bx)
          tma_load_4d(stat_tiles + C::stat_off(i) + bx * (BM * 128), &p.stat[i], &bars->stat_full, bx * 64, m0,
                      head_h, head_b);
      int issued = 0;
      for (int it = 0; it < n_iter; ++it) {
        const int slot = it % C::NSLOT;
        if (!wait_bar(&bars->strm_free[slot], ((it / C::NSLOT) & 1) ^ 1, bars, status)) break;
        mbar_arrive_expect_tx(&bars->strm_full[slot], C::TX_BYTES);
        uint8_t* dst = strm_tiles + slot * C::SLOT_BYTES;
        const int n0 = (t_begin + it) * BN;
#pragma unroll
        for (int i = 0; i < C::NSTRM; ++i)
          for (int bx = 0; bx < C::tile_d(i) / 64; ++bx)
            tma_load_4d(dst + C::strm_off(i) + bx * (BN * 128), &p.strm[i], &bars->strm_full[slot], bx * 64, n0,
                        head_h, head_b);
        if (MODE == FO_BK) {
          const size_t vo = static_cast<size_t>(head) * row_stride(p.n_q) + n0;
          uint8_t* sv = dst + C::STRM_BYTES;
          bulk_load(sv, p.nlc + vo, BN * 4, &bars->strm_full[slot]);
          bulk_load(sv + BN * 4, p.k1 + vo, BN * 4, &bars->strm_full[slot]);
        }
        issued = it + 1;
      }
      // drain: every load issued above must have landed before the CTA may exit
      wait_bar(&bars->stat_full, 0, bars, status);
      for (int it = issued > C::NSLOT ? issued - C::NSLOT : 0; it < issued; ++it) {
        const int slot = it % C::NSLOT;
        const long long start = clock64();
        while (!mbar_try_wait(&bars->strm_full[slot], (it / C::NSLOT) & 1)) {
          if (clock64() - start > kTimeoutCycles) {
            atomicOr(status, FHOB_ERR_TIMEOUT);
            break;
          }
        }
      }
    }
  } else if (warp == MMA_WARP || (warp == MMA_WARP2 && MODE != FO_LSE)) {
    // ================================================= MMA issuers (whole warp runs the loop, one lane issues)
    // One thread cannot issue the products of a tile fast enough, so two warps share them.
    // Backward modes: warp 0 issues the S products and the output products, warp 1 the dP products;
    // warp 1 reuses the dP columns of a stage (they hold dS by then) only after warp 0 has issued
    // the outputs that read them.  Forward modes with an output: warp 0 issues the S products,
    // warp 1 the P V products; warp 0 reuses a stage (it holds P by then) only after warp 1 has
    // issued the product that reads it.  The tensor pipe runs MMAs in the order they arrive.
    constexpr bool kSplitOutputs = C::kForward && MODE != FO_LSE;  // warp 1 issues the outputs
    const int role = warp == MMA_WARP ? 0 : 1;
    if (n_iter > 0) {
      const bool leader = lane == 0;
      auto wait_all = [&](uint64_t* bar, uint32_t parity) {
        return __all_sync(0xffffffffu, wait_bar(bar, parity, bars, status)) != 0;
      };
      auto commit = [&](uint64_t* bar) {
        if (leader) umma_commit(bar);
      };
      constexpr uint32_t idesc_s = umma_idesc_bf16(BM, BN, false, false, F16);
      constexpr uint32_t idesc_o0 = umma_idesc_bf16(BM, C::OUT0_COLS ? C::OUT0_COLS : 64, false, true, F16);  // O | dQ | dK
      constexpr uint32_t idesc_o1 = umma_idesc_bf16(BM, DV, false, true, F16);                                // dV
      constexpr uint32_t idesc_o64 = umma_idesc_bf16(BM, 64, false, true, F16);   // split operands: the hi box alone
      constexpr int kStatBox = BM * 128, kStrmBox = BN * 128;
      constexpr int kLoTile = BN / 4;   // split 16-bit tiles: the lo half starts this many columns after the hi half
      const uint32_t stat_lo = umma_desc_lo(smem_u32(stat_tiles), 16);
      const uint32_t strm_lo = umma_desc_lo(smem_u32(strm_tiles), 16);
      constexpr uint32_t kStat16 = C::stat_off(1) >> 4, kSlot16 = C::SLOT_BYTES >> 4, kStrm16 = C::strm_off(1) >> 4;
      // MN-major view of streamed tile i: leading byte offset = distance between its two 64-column boxes
      auto mn_lo = [&](uint32_t slot_lo, int i) {
        return slot_lo - (1u << 16) + i * kStrm16 + (static_cast<uint32_t>(kStrmBox >> 4) << 16);
      };
      // score product over KD columns (or over the hi/lo boxes of split operands)
      auto scores_mma = [&](auto kd, uint32_t d, uint32_t a, uint32_t b, bool accumulate) {
        if constexpr (SPLIT) fo_gemm_ss_split<kStatBox, kStrmBox>(leader, d, a, b, idesc_s, accumulate);
        else gemm_ss<decltype(kd)::value, kStatBox, kStrmBox>(leader, d, a, b, idesc_s, accumulate);
      };
      // output product, A = 16-bit tile in TMEM; split operands: A_hi . [B_hi | B_lo], then A_lo . B_hi
      auto outputs_mma = [&](uint32_t out, uint32_t a_region, uint32_t b, uint32_t idesc, bool accumulate) {
        gemm_ts<BN>(leader, out, a_region, b, idesc, accumulate);
        if constexpr (SPLIT) gemm_ts<BN>(leader, out, a_region + kLoTile, b, idesc_o64, true);
      };
      using KQ = std::integral_constant<int, DQK>;
      using KV = std::integral_constant<int, DV>;
      bool ok = wait_all(&bars->stat_full, 0);

      if (kSplitOutputs) {
        for (int it = 0; ok && it < n_iter; ++it) {
          const int slot = it % C::NSLOT, stage = it & 1;
          const uint32_t acc = tmem_base + C::OUT_COLS + stage * C::STAGE_COLS;
          const uint32_t sl = strm_lo + slot * kSlot16;
          if (role == 0) {
            if (it >= 2) ok = wait_all(&bars->go[stage], ((it - 2) >> 1) & 1);
            ok = ok && wait_all(&bars->strm_full[slot], (it / C::NSLOT) & 1);
            if (!ok) break;
            tc_fence_after();
            scores_mma(KQ{}, acc, stat_lo, sl, false);  // S
            commit(&bars->s_full[stage]);
          } else {
            ok = wait_all(&bars->p_full[stage], (it >> 1) & 1) && wait_all(&bars->strm_full[slot], (it / C::NSLOT) & 1);
            if (!ok) break;
            tc_fence_after();
            outputs_mma(tmem_base, acc, mn_lo(sl, 1), idesc_o0, it > 0);  // O += P . V
            commit(&bars->strm_free[slot]);
            if (MODE == FO_ONE) commit(&bars->o_done);
            if (leader) mbar_arrive(&bars->go[stage]);
          }
        }
      } else if (role == 1) {
        for (int it = 0; ok && it < n_iter; ++it) {
          const int slot = it % C::NSLOT, stage = it & 1;
          if (it >= 2) ok = wait_all(&bars->go[stage], ((it - 2) >> 1) & 1);
          ok = ok && wait_all(&bars->strm_full[slot], (it / C::NSLOT) & 1);
          if (!ok) break;
          tc_fence_after();
          const uint32_t acc = tmem_base + C::OUT_COLS + stage * C::STAGE_COLS;
          const uint32_t sl = strm_lo + slot * kSlot16;
          scores_mma(KV{}, acc + BN, stat_lo + kStat16, sl + kStrm16, false);  // dP
          commit(&bars->s_full[stage]);
        }
      } else {
        auto scores = [&](int it) -> bool {
          const int slot = it % C::NSLOT, stage = it & 1;
          if (!wait_all(&bars->strm_full[slot], (it / C::NSLOT) & 1)) return false;
          if (MODE == FO_LSE && !wait_all(&bars->s_free[stage], ((it >> 1) & 1) ^ 1)) return false;
          tc_fence_after();
          const uint32_t acc = tmem_base + C::OUT_COLS + stage * C::STAGE_COLS;
          const uint32_t sl = strm_lo + slot * kSlot16;
          scores_mma(KQ{}, acc, stat_lo, sl, false);  // S
          commit(&bars->s_full[stage]);
          if (MODE == FO_LSE) commit(&bars->strm_free[slot]);
          return true;
        };

        ok = ok && scores(0);
        for (int it = 0; ok && it < n_iter; ++it) {
          if (it + 1 < n_iter) {
            ok = scores(it + 1);
            if (!ok) break;
          }
          if (MODE != FO_LSE) {
            const int slot = it % C::NSLOT, stage = it & 1;
            ok = wait_all(&bars->p_full[stage], (it >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + C::OUT_COLS + stage * C::STAGE_COLS;
            const uint32_t sl = strm_lo + slot * kSlot16;
            const bool accum = it > 0;
            if (MODE == FO_ONE) {
              outputs_mma(tmem_base, acc, mn_lo(sl, 1), idesc_o0, accum);                     // O  += P . V
              commit(&bars->o_done);
            } else if (MODE == FO_BQ) {
              outputs_mma(tmem_base, acc + BN, mn_lo(sl, 0), idesc_o0, accum);                // dQ += dS . K
            } else {
              outputs_mma(tmem_base + C::OUT0_COLS, acc, mn_lo(sl, 1), idesc_o1, accum);      // dV += P^T . dO
              outputs_mma(tmem_base, acc + BN, mn_lo(sl, 0), idesc_o0, accum);                // dK += dS^T . Q
            }
            commit(&bars->strm_free[slot]);
            if (C::NACC == 2 && leader) mbar_arrive(&bars->go[stage]);
          }
        }
      }
      if (ok) {
        if (MODE != FO_LSE && role == (kSplitOutputs ? 1 : 0)) commit(&bars->out_full);
      } else {
        // abort path: no tcgen05.mma may still be reading shared memory or TMEM at exit
        commit(&bars->teardown[role]);
        const long long start = clock64();
        while (!mbar_try_wait(&bars->teardown[role], 0)) {
          if (clock64() - start > kTimeoutCycles) break;
        }
      }
    }
  } else if (warp >= EW_WARP0) {
    // ================================================= elementwise warps
    const int quad = warp & 3, half = (warp - EW_WARP0) >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int g_row = m0 + row;  // stationary row of this thread
    const float sl2 = p.scale * kLog2e;
    float r_nlc = 0.f, r_k1 = 0.f;
    if (kQStat && g_row < p.n_q) {
      if (MODE == FO_BQ) {
        const size_t vi = static_cast<size_t>(head) * row_stride(p.n_q) + g_row;
        r_nlc = p.nlc[vi];
        r_k1 = p.k1[vi];
      }
    }
    // visible streamed index range of this thread's row
    int lo, hi;
    if (kQStat) {
      lo = 0;
      hi = p.n_k - 1;
      if (p.causal && g_row + off < hi) hi = g_row + off;
      if (p.window > 0 && g_row + off - p.window + 1 > 0) lo = g_row + off - p.window + 1;
    } else {
      lo = p.causal ? g_row - off : 0;
      if (lo < 0) lo = 0;
      hi = p.n_q - 1;
      if (p.window > 0 && g_row - off + p.window - 1 < hi) hi = g_row - off + p.window - 1;
    }
    float run_m = -INFINITY, run_l = 0.f;  // LSE: running maximum (log2 domain) and sum
    bool ok = true;

    for (int it = 0; it < n_iter; ++it) {
      const int n0 = (t_begin + it) * BN;
      const int stage = it & 1;
      bool masked = n0 + BN > n_strm;
      if (p.causal) {
        if (kQStat) masked = masked || (n0 + BN - 1 > m0 + off);
        else masked = masked || (n0 + off < m0 + BM - 1);
        if (p.window > 0) {
          if (kQStat) masked = masked || (m0 + BM - 1 + off - n0 >= p.window);
          else masked = masked || (n0 + BN - 1 + off - m0 >= p.window);
        }
      }
      const int col_base = n0 + half * CPT;
      uint32_t sv = 0;
      if (MODE == FO_BK) {
        // the slot's vectors were written by the TMA unit: observe its barrier before reading them
        const int slot = it % C::NSLOT;
        ok = __all_sync(0xffffffffu, wait_bar(&bars->strm_full[slot], (it / C::NSLOT) & 1, bars, status));
        if (!ok) break;
        sv = smem_u32(strm_tiles + slot * C::SLOT_BYTES + C::STRM_BYTES) + half * CPT * 4;
      }
      ok = __all_sync(0xffffffffu, wait_bar(&bars->s_full[stage], (it >> 1) & 1, bars, status));
      if (!ok) break;
      tc_fence_after();
      const uint32_t acc = tmem_base + lane_base + C::OUT_COLS + stage * C::STAGE_COLS + half * CPT;

      if (MODE == FO_LSE) {
        // online log-sum-exp over this thread's 64 columns of the tile, in the log2 domain
        float tile_m = -INFINITY;
        uint32_t x[2][32];
        tmem_ld32(acc, x[0]);
        tmem_ld32(acc + 32, x[1]);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&bars->s_free[stage]);
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int idx = col_base + 32 * c + j;
            float y = __uint_as_float(x[c][j]) * sl2;
            if (masked && !(idx >= lo && idx <= hi)) y = -INFINITY;
            x[c][j] = __float_as_uint(y);
            tile_m = fmaxf(tile_m, y);
          }
        const float new_m = fmaxf(run_m, tile_m);
        if (new_m != -INFINITY) {
          float2 sum = make_float2(0.f, 0.f);
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int j = 0; j < 32; j += 2)
              sum = __fadd2_rn(sum, make_float2(ex2(__uint_as_float(x[c][j]) - new_m),
                                                ex2(__uint_as_float(x[c][j + 1]) - new_m)));
          run_l = run_l * ex2(run_m - new_m) + (sum.x + sum.y);
          run_m = new_m;
        }
      } else if (MODE == FO_ONE) {
        // single-sweep forward: online softmax with a lazily updated reference maximum.  P is
        // formed against m_used, which follows the running row maximum only when that has grown
        // by more than 8 (P stays below 2^8); O and the row sum are rescaled on those occasions.
        uint32_t xx[2][32], w[2][16], w_lo[2][16];
        tmem_ld32(acc, xx[0]);
        tmem_ld32(acc + 32, xx[1]);
        tmem_wait_ld();
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float2 y = __fmul2_rn(f2(xx[c][j], xx[c][j + 1]), make_float2(sl2, sl2));
            if (masked) {
              const int idx = col_base + 32 * c + j;
              y.x = (idx >= lo && idx <= hi) ? y.x : -INFINITY;
              y.y = (idx + 1 >= lo && idx + 1 <= hi) ? y.y : -INFINITY;
            }
            xx[c][j] = __float_as_uint(y.x);
            xx[c][j + 1] = __float_as_uint(y.y);
            mx[(j >> 1) & 3] = fmaxf(mx[(j >> 1) & 3], fmaxf(y.x, y.y));
          }
        float tile_m = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        // the row's maximum over both column halves (the partner warp owns the other 64 columns)
        bars->red[it & 1][half][row] = tile_m;
        mbar_arrive(&bars->pair[quad]);
        ok = __all_sync(0xffffffffu, wait_bar(&bars->pair[quad], it & 1, bars, status));
        if (!ok) break;
        tile_m = fmaxf(tile_m, bars->red[it & 1][half ^ 1][row]);
        const bool need = tile_m > run_m + 8.f;   // run_m holds m_used; true for the first finite maximum
        if (it > 0 && __any_sync(0xffffffffu, need)) {
          // O is idle once the previous tile's P V has finished; the next one waits for this tile's P
          ok = __all_sync(0xffffffffu, wait_bar(&bars->o_done, (it - 1) & 1, bars, status));
          if (!ok) break;
          tc_fence_after();
          const float alpha = (need && run_m != -INFINITY) ? ex2(run_m - tile_m) : 1.f;
#pragma unroll
          for (int ch = 0; ch < C::OUT0_COLS / 64; ++ch) {
            uint32_t v[32], lo16[16], hi16[16];
            const uint32_t addr = tmem_base + lane_base + half * (C::OUT0_COLS / 2) + 32 * ch;
            tmem_ld32(addr, v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              lo16[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
              hi16[j] = __float_as_uint(__uint_as_float(v[16 + j]) * alpha);
            }
            tmem_st16(addr, lo16);
            tmem_st16(addr + 16, hi16);
          }
          tmem_wait_st();
          run_l *= alpha;
        }
        if (need) run_m = tile_m;
        const float neg_m = run_m == -INFINITY ? 0.f : -run_m;
        float2 sum = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float2 d = __fadd2_rn(f2(xx[c][j], xx[c][j + 1]), make_float2(neg_m, neg_m));
            const float2 pr = make_float2(ex2(d.x), ex2(d.y));
            sum = __fadd2_rn(sum, pr);
            if constexpr (SPLIT) fo_split_pack(pr.x, pr.y, w[c][j / 2], w_lo[c][j / 2]);
            else w[c][j / 2] = pack16<F16>(pr.x, pr.y);
          }
        run_l += sum.x + sum.y;
        // the thread's 64 score columns take its 32 packed columns of P (split: then 32 of the lo halves)
        tmem_st16(acc, w[0]);
        tmem_st16(acc + 16, w[1]);
        if constexpr (SPLIT) {
          tmem_st16(acc + 32, w_lo[0]);
          tmem_st16(acc + 48, w_lo[1]);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&bars->p_full[stage]);
      } else {
        uint32_t s[32], dp[32], w_p[16], w_ds[16], w_p_lo[16], w_ds_lo[16];
        tmem_ld32(acc, s);
        tmem_ld32(acc + BN, dp);
        tmem_wait_ld();
#pragma unroll
        for (int j4 = 0; j4 < 8; ++j4) {
          float c_nlc[4], c_k1[4];
          if (kQStat) {
#pragma unroll
            for (int e = 0; e < 4; ++e) { c_nlc[e] = r_nlc; c_k1[e] = r_k1; }
          } else {
            load4(sv + (4 * j4) * 4, c_nlc);
            load4(sv + (BN + 4 * j4) * 4, c_k1);
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int j = 4 * j4 + 2 * h;
            const float2 arg = __ffma2_rn(f2(s[j], s[j + 1]), make_float2(sl2, sl2),
                                          make_float2(c_nlc[2 * h], c_nlc[2 * h + 1]));
            float2 pr = make_float2(ex2(arg.x), ex2(arg.y));
            const float2 dpp = __fadd2_rn(f2(dp[j], dp[j + 1]), make_float2(c_k1[2 * h], c_k1[2 * h + 1]));
            float2 ds = __fmul2_rn(pr, dpp);
            if (masked) {
              const int idx = col_base + j;
              const bool ok0 = idx >= lo && idx <= hi, ok1 = idx + 1 >= lo && idx + 1 <= hi;
              pr.x = ok0 ? pr.x : 0.f; pr.y = ok1 ? pr.y : 0.f;
              ds.x = ok0 ? ds.x : 0.f; ds.y = ok1 ? ds.y : 0.f;
            }
            if constexpr (SPLIT) {
              fo_split_pack(ds.x, ds.y, w_ds[j / 2], w_ds_lo[j / 2]);
              if (MODE == FO_BK) fo_split_pack(pr.x, pr.y, w_p[j / 2], w_p_lo[j / 2]);
            } else {
              w_ds[j / 2] = pack16<F16>(ds.x, ds.y);
              if (MODE == FO_BK) w_p[j / 2] = pack16<F16>(pr.x, pr.y);
            }
          }
        }
        tmem_st16(acc + BN, w_ds);
        if (MODE == FO_BK) tmem_st16(acc, w_p);
        if constexpr (SPLIT) {
          tmem_st16(acc + BN + 16, w_ds_lo);
          if (MODE == FO_BK) tmem_st16(acc + 16, w_p_lo);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&bars->p_full[stage]);
      }
    }

    // ---- results
    if (MODE == FO_LSE) {
      if (half == 1) {
        bars->red[0][0][row] = run_m;
        bars->red[0][1][row] = run_l;
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (half == 0 && ok && g_row < p.n_q) {
        const float m1 = bars->red[0][0][row], l1 = bars->red[0][1][row];
        const float m = fmaxf(run_m, m1);
        float lse = -INFINITY;
        if (m != -INFINITY) {
          const float l = run_l * ex2(run_m - m) + l1 * ex2(m1 - m);
          lse = (m + log2f(l)) * 0.6931471805599453f;
        }
        p.lse_out[static_cast<size_t>(head) * p.n_q + g_row] = lse;
      }
    } else {
      float inv_l = 1.f;
      if (MODE == FO_ONE) {
        // row sum over both column halves; L = m_used + log(sum), O = accumulator / sum
        asm volatile("bar.sync 1, 256;" ::: "memory");  // every reader of the per-tile maxima is done
        bars->red[0][half][row] = run_l;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const float l = run_l + bars->red[0][half ^ 1][row];
        inv_l = l > 0.f ? 1.f / l : 0.f;
        if (half == 0 && ok && g_row < p.n_q)
          p.lse_out[static_cast<size_t>(head) * p.n_q + g_row] =
              l > 0.f ? (run_m + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
      if (n_iter > 0) ok = ok && __all_sync(0xffffffffu, wait_bar(&bars->out_full, 0, bars, status));
      tc_fence_after();
      if (ok) {
        // result o: `width` columns starting at TMEM column col0; dS was stored without the scale; the
        // single-sweep forward divides by the row sum here
        auto store_out = [&](auto width, int d_mem, uint32_t col0, uint16_t* base, float mul) {
          constexpr int DO = decltype(width)::value;   // columns of the accumulator; d_mem <= DO of them exist in memory
          uint16_t* dst = base + (static_cast<size_t>(head) * n_stat + (g_row < n_stat ? g_row : 0)) * d_mem + half * (DO / 2);
#pragma unroll
          for (int ch = 0; ch < DO / 32; ++ch) {
            uint32_t v[16];
            if (n_iter > 0) {
              tmem_ld16(tmem_base + lane_base + col0 + half * (DO / 2) + 16 * ch, v);
              tmem_wait_ld();
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = 0u;
            }
            if (g_row < n_stat) {
              uint32_t w[8];
#pragma unroll
              for (int j = 0; j < 8; ++j)
                w[j] = pack16<F16>(__uint_as_float(v[2 * j]) * mul, __uint_as_float(v[2 * j + 1]) * mul);
              uint4* d4 = reinterpret_cast<uint4*>(dst + 16 * ch);
              const int c0 = half * (DO / 2) + 16 * ch;   // head dims are multiples of 8: 16-byte pieces are whole
              if (c0 + 8 <= d_mem) d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
              if (c0 + 16 <= d_mem) d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
          }
        };
        // split operands: 64 fp32 columns, the sum of the two 64-column halves of the accumulator
        auto store_out_split = [&](int d_mem, uint32_t col0, uint16_t* base16, float mul) {
          float* dst = reinterpret_cast<float*>(base16) +
                       (static_cast<size_t>(head) * n_stat + (g_row < n_stat ? g_row : 0)) * d_mem + half * 32;
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            uint32_t a[16], b[16];
            if (n_iter > 0) {
              tmem_ld16(tmem_base + lane_base + col0 + half * 32 + 16 * ch, a);
              tmem_ld16(tmem_base + lane_base + col0 + 64 + half * 32 + 16 * ch, b);
              tmem_wait_ld();
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) a[j] = b[j] = 0u;
            }
            if (g_row < n_stat) {
              float4* d4 = reinterpret_cast<float4*>(dst + 16 * ch);
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (half * 32 + 16 * ch + 4 * j + 4 <= d_mem)   // head dims are multiples of 4: float4 pieces are whole
                d4[j] = make_float4((__uint_as_float(a[4 * j]) + __uint_as_float(b[4 * j])) * mul,
                                    (__uint_as_float(a[4 * j + 1]) + __uint_as_float(b[4 * j + 1])) * mul,
                                    (__uint_as_float(a[4 * j + 2]) + __uint_as_float(b[4 * j + 2])) * mul,
                                    (__uint_as_float(a[4 * j + 3]) + __uint_as_float(b[4 * j + 3])) * mul);
            }
          }
        };
        const float mul0 = MODE == FO_ONE ? inv_l : p.scale;
        if constexpr (SPLIT) {
          store_out_split(p.d_out0, 0, p.out0, mul0);
          if (C::NOUT == 2) store_out_split(p.d_out1, C::OUT0_COLS, p.out1, 1.f);
        } else {
          store_out(std::integral_constant<int, (C::OUT0_COLS ? C::OUT0_COLS : 64)>{}, p.d_out0, 0, p.out0, mul0);
          if constexpr (C::NOUT == 2) store_out(std::integral_constant<int, DV>{}, p.d_out1, C::OUT0_COLS, p.out1, 1.f);
        }
      }
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int MODE, int DQK, int DV, bool F16, bool SPLIT = false>
int fo_launch(const FhobProblem& p, FoParams& tp, cudaStream_t s) {
  using C = FoCfg<MODE, DQK, DV>;
  const void* q_side[2] = {p.q, p.d_o};
  const void* k_side[2] = {p.k, p.v};
  if (SPLIT) {
    // the bf16 hi/lo copies the caller of this function left in the workspace
    SplitBuffers sb = split_buffers(p);
    q_side[0] = sb.q; q_side[1] = sb.d_o;
    k_side[0] = sb.k; k_side[1] = sb.v;
  }
  // head dims below the tile widths: the boxes reach past the end of a row and are zero-filled there
  const int d_mem[2] = {SPLIT ? 128 : p.d, SPLIT ? 128 : head_dim_v(p)};
  // where each input lives: the caller's layout, or contiguous (always so for the split copies)
  const int q_ids[2] = {kTenQ, kTenDO}, k_ids[2] = {kTenK, kTenV};
  auto view = [&](int id, int n_rows, int d) {
    return SPLIT ? contiguous_view(p.bh, n_rows, d) : tensor_view(p, id, n_rows, d);
  };
  int st = FHOB_OK;
  if (MODE != FO_BK) {
    for (int i = 0; i < C::NSTAT && st == FHOB_OK; ++i)
      st = make_map(&tp.stat[i], q_side[i], view(q_ids[i], p.n_q, d_mem[i]), p.n_q, d_mem[i], BM, F16);
    for (int i = 0; i < C::NSTRM && st == FHOB_OK; ++i)
      st = make_map(&tp.strm[i], k_side[i], view(k_ids[i], p.n_k, d_mem[i]), p.n_k, d_mem[i], C::BN, F16);
  } else {
    for (int i = 0; i < C::NSTAT && st == FHOB_OK; ++i)
      st = make_map(&tp.stat[i], k_side[i], view(k_ids[i], p.n_k, d_mem[i]), p.n_k, d_mem[i], BM, F16);
    for (int i = 0; i < C::NSTRM && st == FHOB_OK; ++i)
      st = make_map(&tp.strm[i], q_side[i], view(q_ids[i], p.n_q, d_mem[i]), p.n_q, d_mem[i], C::BN, F16);
  }
  if (st != FHOB_OK) return st;
  tp.heads = (!SPLIT && p.layout) ? p.layout->heads : p.bh;
  tp.d_out0 = MODE == FO_ONE ? head_dim_v(p) : p.d;   // columns in memory of O | dQ | dK
  tp.d_out1 = head_dim_v(p);                          // dV
  tp.n_q = p.n_q; tp.n_k = p.n_k; tp.causal = p.causal; tp.window = p.window; tp.scale = p.scale;
  const int n_stat = MODE == FO_BK ? p.n_k : p.n_q;
  tp.tiles_per_head = (n_stat + BM - 1) / BM;
  constexpr auto kernel = fo_kernel<MODE, DQK, DV, F16, SPLIT>;
  {
    const int st_attr = allow_smem(kernel, C::SMEM_BYTES);
    if (st_attr != FHOB_OK) return st_attr;
  }
  const long long blocks = static_cast<long long>(tp.tiles_per_head) * p.bh;
  if (blocks > 0x7fffffffLL) return FHOB_ERR_SHAPE;
  kernel<<<static_cast<unsigned>(blocks), NTHREADS, C::SMEM_BYTES, s>>>(tp);
  FHOB_CUDA_OK(cudaGetLastError());
  return FHOB_OK;
}

int check_device() {
  static thread_local int checked_dev = -1;
  int dev = 0;
  FHOB_CUDA_OK(cudaGetDevice(&dev));
  if (dev != checked_dev) {
    int major = 0;
    FHOB_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) return FHOB_ERR_ARCH;
    checked_dev = dev;
  }
  return FHOB_OK;
}

template <int DQK, int DV, bool F16, bool SPLIT = false>
int forward_impl(const FhobProblem& p, void* o_out, float* lse_out, int* status, cudaStream_t s) {
  FoParams tp;
  memset(&tp, 0, sizeof(tp));
  tp.status = status;
  tp.lse_out = lse_out;
  tp.out0 = static_cast<uint16_t*>(o_out);
  // no O wanted: the scores alone, reduced to the logsumexp (no tile of the second head dim is touched)
  return o_out ? fo_launch<FO_ONE, DQK, DV, F16, SPLIT>(p, tp, s) : fo_launch<FO_LSE, DQK, DQK, F16, SPLIT>(p, tp, s);
}

template <int DQK, int DV, bool F16, bool SPLIT = false>
int backward_impl(const FhobProblem& p, void* dq, void* dk, void* dv, cudaStream_t s) {
  RowVectors rv = row_vectors(p);
  FoParams tp;
  memset(&tp, 0, sizeof(tp));
  tp.status = rv.status;
  tp.nlc = rv.nlc;
  tp.k1 = rv.k1;
  tp.out0 = static_cast<uint16_t*>(dq);
  int st = fo_launch<FO_BQ, DQK, DV, F16, SPLIT>(p, tp, s);
  if (st != FHOB_OK) return st;
  tp.out0 = static_cast<uint16_t*>(dk);
  tp.out1 = static_cast<uint16_t*>(dv);
  return fo_launch<FO_BK, DQK, DV, F16, SPLIT>(p, tp, s);
}

// One warp waits on an mbarrier nothing ever arrives on: exercises the give-up branch of wait_bar.
struct ExpireBars {
  uint64_t bar;
  int abort_flag;
};
__global__ void expire_wait_kernel(int* status) {
  __shared__ ExpireBars b;
  if (threadIdx.x == 0) {
    mbar_init(&b.bar, 1);
    b.abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  wait_bar(&b.bar, 0, &b, status);
}

}  // namespace

int tc_selftest_expired_wait(int* status, cudaStream_t s) {
  expire_wait_kernel<<<1, 32, 0, s>>>(status);
  FHOB_CUDA_OK(cudaGetLastError());
  return FHOB_OK;
}

// 16-bit problems with head dims in {64, 128} (any combination), and fp32 problems with both head
// dims 64 whose workspace holds the bf16 hi/lo copies (see tc_split_supported)
bool tc_first_order_supported(const FhobProblem& p) { return tc_supported(p); }

namespace {
template <bool F16, class Fn>
int by_dims(const FhobProblem& p, Fn&& fn) {
  const int dv = head_dim_v(p);
  // tile widths: the head dims rounded up to 64 or 128
  if (p.d <= 64) return dv <= 64 ? fn(std::integral_constant<int, 64>{}, std::integral_constant<int, 64>{})
                                 : fn(std::integral_constant<int, 64>{}, std::integral_constant<int, 128>{});
  return dv <= 64 ? fn(std::integral_constant<int, 128>{}, std::integral_constant<int, 64>{})
                  : fn(std::integral_constant<int, 128>{}, std::integral_constant<int, 128>{});
}
}  // namespace

int tc_forward(const FhobProblem& p, void* o_out, float* lse_out, int* status, cudaStream_t s) {
  if (!tc_first_order_supported(p)) return FHOB_ERR_SHAPE;
  int st = check_device();
  if (st != FHOB_OK) return st;
  if (p.dtype == FHOB_F32) {
    st = tc_split_inputs(p, s, kSplitQ | kSplitK | (o_out ? kSplitV : 0));
    if (st != FHOB_OK) return st;
    return forward_impl<128, 128, false, true>(p, o_out, lse_out, status, s);
  }
  if (p.dtype == FHOB_F16)
    return by_dims<true>(p, [&](auto dqk, auto dv) {
      return forward_impl<decltype(dqk)::value, decltype(dv)::value, true>(p, o_out, lse_out, status, s);
    });
  return by_dims<false>(p, [&](auto dqk, auto dv) {
    return forward_impl<decltype(dqk)::value, decltype(dv)::value, false>(p, o_out, lse_out, status, s);
  });
}

int tc_backward(const FhobProblem& p, void* dq, void* dk, void* dv, cudaStream_t s) {
  if (!tc_first_order_supported(p)) return FHOB_ERR_SHAPE;
  int st = check_device();
  if (st != FHOB_OK) return st;
  if (p.dtype == FHOB_F32) {
    st = tc_split_inputs(p, s, kSplitQ | kSplitK | kSplitV | kSplitDO);
    if (st != FHOB_OK) return st;
    return backward_impl<128, 128, false, true>(p, dq, dk, dv, s);
  }
  if (p.dtype == FHOB_F16)
    return by_dims<true>(p, [&](auto dqk, auto dvv) {
      return backward_impl<decltype(dqk)::value, decltype(dvv)::value, true>(p, dq, dk, dv, s);
    });
  return by_dims<false>(p, [&](auto dqk, auto dvv) {
    return backward_impl<decltype(dqk)::value, decltype(dvv)::value, false>(p, dq, dk, dv, s);
  });
}

}  // namespace fhob
