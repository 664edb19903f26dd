// Tensor-core kernels of the double-backward attention operator for sm_100a:
// TMA tile loads -> tcgen05.mma with fp32 accumulators in TMEM -> tcgen05.ld
// into registers for the elementwise math -> (passes 3, 4) 16-bit tiles (bf16
// or f16, the storage type) written back to TMEM and used as the A operand of
// the output products.
//
// One kernel template covers the four passes (reference: passes 1-3 are the
// three key loops of bwdbwd_kernel_stage1, fhog/triton_bwdbwd.py:178-313;
// pass 4 is bwdbwd_kernel_stage2, :321-535) and the sweep that replaces passes
// 1 and 2 in the operator (FUSED: both row statistics from one recomputation).  A CTA owns BM = 128 "stationary"
// rows of one head (queries in passes 1-3, keys in pass 4) which become the 128
// TMEM lanes, and streams BN-row tiles of the other side:
//
//   score-shaped accumulators (128 x BN fp32 each, K-major smem x K-major smem):
//     group A:  [S | stat0.strm1^T] = stat0 . [strm0 ; strm1]^T     A2 += stat1 . strm0^T
//     group B:  [dP | X] = stat2 . [strm2 ; strm3]^T      (pass 4: dP = stat2.strm2^T, X = stat3.strm2^T)
//   output accumulators (128 x D fp32 each, A = bf16 tile in TMEM, B = streamed tile read MN-major):
//     pass 3: ddO += ddP . V + P . ddV   (after group A)     dQ2 += dS . ddK + dS2 . K     (after group B)
//     pass 4: dV2 += ddP^T . dO          (after group A)     dK2 += dS^T . ddQ + dS2^T . Q (after group B)
//
// Warp roles (384 threads): warps 0, 1 and 3 = MMA issuers (one lane each; warp 0 also allocates
// TMEM), warp 2 = TMA producer (one lane), warps 4-11 elementwise (warp w owns TMEM lanes
// 32*(w%4).., column half (w-4)/4).  The products of a tile fall into two chains that never touch
// the same TMEM columns - chain 1: group A -> P, ddP -> ddO | dV2; chain 2: group B -> dS, dS2 ->
// dQ2 | dK2 - so each chain has its own issuing warp, on its own warp scheduler.  Issuing a
// tcgen05.mma keeps a thread busy for about 51 cycles and the elementwise warps of the same
// scheduler delay it further; one thread cannot feed 64-cycle products under that load.  For the
// same reason, in passes 1 and 2 the second product of group A (A2 += stat1 . strm0^T) is issued
// by a third warp, strictly behind chain 1's stacked product (the tensor pipe runs MMAs in the
// order they arrive, so the accumulation order stays fixed and results stay bit-reproducible).
//   passes 1, 2: two score stages in TMEM; the MMA warp runs one tile ahead.
//   passes 3, 4: TMEM is full with one stage (2*D + 4*64 columns), so the tile is pipelined in
//   two halves instead: while the elementwise warps turn group A into P / ddP, the tensor core
//   computes group B; while they turn group B into dS / dS2, it runs the group-A outputs and
//   group A of the next tile.  The bf16 tiles overwrite their own accumulators in place.
// Every mbarrier wait is bounded: when it runs out the CTA raises the status word, drains and exits.
#include <type_traits>

#include "tc_common.cuh"

// pass 3: start the first elementwise half when S alone is complete (see ew_half_a)
#ifndef FHOB_EARLY_S
#define FHOB_EARLY_S 1
#endif

namespace fhob {
namespace {


template <int PASS, int DQK, int DV, int BN>
struct Cfg {
  static constexpr int NSTAT = PASS == 1 ? 2 : (PASS == 4 ? 4 : 3);
  static constexpr int NSTRM = PASS == 1 ? 2 : (PASS == 4 ? 3 : 4);
  static constexpr int NACC = PASS == 1 ? 2 : 4;
  static constexpr int NOUT = PASS >= 3 ? 2 : 0;
  // Two head dims (jax_refs/flash_impl.py:381-389 uses d_in != d_out): Q, K, ddQ, ddK and the
  // results dQ2, dK2 have DQK columns; V, ddV, dO and the results ddO, dV2 have DV columns.  In
  // every pass the first two stationary and the first two streamed tiles are of the first kind
  // (passes 1-3: Q, ddQ | dO and K, ddK | V, ddV; pass 4: K, ddK | V, ddV and Q, ddQ | dO).
  __host__ __device__ static constexpr int tile_d(int i) { return i < 2 ? DQK : DV; }
  static constexpr int OUT0_COLS = NOUT ? DQK : 0;   // dQ2 | dK2
  static constexpr int OUT1_COLS = NOUT ? DV : 0;    // ddO | dV2
  static constexpr int OUT_COLS = OUT0_COLS + OUT1_COLS;
  static constexpr int STAGE_COLS = NACC * BN;
  // score stages in TMEM: two for the reducing passes, one (pipelined in halves) for passes 3, 4
  static constexpr int NSS = PASS <= 2 ? ((TMEM_COLS - OUT_COLS) / STAGE_COLS >= 2 ? 2 : 1) : 1;
  __host__ __device__ static constexpr int stat_bytes(int i) { return BM * tile_d(i) * 2; }
  __host__ __device__ static constexpr int strm_bytes(int i) { return BN * tile_d(i) * 2; }
  __host__ __device__ static constexpr int stat_off(int i) { return i == 0 ? 0 : stat_off(i - 1) + stat_bytes(i - 1); }
  static constexpr int STAT_BYTES = stat_off(NSTAT);
  // Streamed tiles 2p and 2p+1 form a pair (same head dim) whose 64-column boxes interleave in
  // shared memory (box b of tile 2p, box b of tile 2p+1, box b+1 of tile 2p, ...), so that one
  // K-major operand descriptor can cover both tiles stacked as 2*BN rows: products that share
  // their A operand (S and Q.ddK^T; dP and X) are then issued as one MMA with N = 2*BN.  A
  // tcgen05.mma occupies the tensor pipe for max(N/2, ~50) cycles on B200 (measured), so two
  // N = 64 products cost 104 cycles where one N = 128 product costs 64.  An unpaired last tile
  // keeps the compact layout.
  __host__ __device__ static constexpr bool paired(int i) { return (i / 2) * 2 + 1 < NSTRM; }
  __host__ __device__ static constexpr int pair_off(int pr) {  // byte offset of the pair's first box
    return pr == 0 ? 0 : pair_off(pr - 1) + strm_bytes(2 * (pr - 1)) * (paired(2 * (pr - 1)) ? 2 : 1);
  }
  __host__ __device__ static constexpr int strm_base(int i) {
    return pair_off(i / 2) + (paired(i) ? (i % 2) * BN * 128 : 0);
  }
  __host__ __device__ static constexpr int strm_box(int i) { return paired(i) ? 2 * BN * 128 : BN * 128; }
  static constexpr int STRM_BYTES = pair_off((NSTRM + 1) / 2);   // all streamed tiles of a slot
  // pass 4: the four per-query constant vectors of the streamed queries travel with the slot
  static constexpr int STATS_BYTES = PASS == 4 ? 4 * BN * 4 : 0;
  static constexpr int SLOT_BYTES = STRM_BYTES + STATS_BYTES;
  static constexpr int NSLOT_FIT = (SMEM_LIMIT - SMEM_TAIL - STAT_BYTES) / SLOT_BYTES;
  static constexpr int NSLOT = NSLOT_FIT > 4 ? 4 : NSLOT_FIT;
  static constexpr int SMEM_BYTES = STAT_BYTES + NSLOT * SLOT_BYTES + SMEM_TAIL;
  static_assert(NSS * STAGE_COLS + OUT_COLS <= TMEM_COLS, "TMEM budget");
  static_assert(NSLOT >= 2, "need two streamed slots");
  static_assert((DQK == 64 || DQK == 128) && (DV == 64 || DV == 128), "head dims");
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 128, "streamed tile");
  static_assert(PASS <= 2 || BN == 64, "passes 3 and 4 are written for 64-row streamed tiles");
};

struct TcParams {
  CUtensorMap stat[4];
  CUtensorMap strm[4];
  const float* nlc;  // -L*log2(e)
  const float* k1;   // -D
  float* ndd;        // -dd           (written by pass 1)
  float* k23;        // -D*dd - b     (written by pass 2)
  uint16_t* out0;  // 16-bit elements: bf16 or f16
  uint16_t* out1;
  int* status;
  int n_q, n_k, causal, window, tiles_per_head;
  int heads;            // heads per batch entry of the input tensor maps (4-D: columns, rows, head, batch)
  int d_out0, d_out1;   // columns of the two results in memory (<= the tile widths DQK, DV; see launch)
  float scale;
};


struct Bars {
  uint64_t stat_full;
  uint64_t strm_full[4];
  uint64_t strm_free[4];
  uint64_t s_full[2];   // passes 1, 2: per score stage; passes 3, 4: [0] = group A done, [1] = group B done
  uint64_t s_free[2];   // passes 1, 2: stage consumed by the elementwise warps
  uint64_t p_full[2];   // passes 3, 4: [0] = P/ddP written, [1] = dS/dS2 written
  uint64_t out_full;
  uint64_t s_ready;      // passes 3, 4: the stacked product [S | Q.ddK^T] of a tile has finished
  uint64_t chain_go;     // passes 3, 4: chain 1 has issued its products of this round (chain 2 may follow)
  uint64_t teardown[3];
  uint64_t a2_go;        // chain 1 has issued the stacked product of a tile: the A2 product may follow
  uint32_t tmem_base;
  int abort_flag;
  float red[BM];
};
static_assert(sizeof(Bars) <= SMEM_TAIL, "tail");



struct EwCtx {
  float scale, sl2;
  float r_nlc, r_k1, r_ndd, r_k23;  // constants of this thread's query row (passes 1-3)
  uint32_t sv;                      // pass 4: shared-memory address of the slot's [nlc|ndd|k1|k23][64] block
  int lo, hi;                       // visible streamed index range of this thread's row
};


// Passes 1 and 2: row reductions over one streamed tile.  acc = TMEM address of the stage (lane
// and column-half offset included); col_base = streamed index of the thread's first column.

// FUSED (pass 2 only): accumulates r[0] = sum P A2, r[1] = sum P X, r[2] = sum dP P A2, from which
// both dd and b follow at the end of the pass without dd being known while the tiles stream by.
// FUSED == 2 also accumulates r[3] = sum P dP = D, for callers that do not pass O.
template <int PASS, int BN, bool MASKED, int FUSED>
__device__ __forceinline__ void ew_reduce(uint32_t acc, int col_base, const EwCtx& c, float2 (&r)[4]) {
  float2& rowacc = r[0];
  constexpr int CH = BN / 32;
  const float2 sl2 = make_float2(c.sl2, c.sl2), nlc = make_float2(c.r_nlc, c.r_nlc);
  const float2 scale = make_float2(c.scale, c.scale), ndd = make_float2(c.r_ndd, c.r_ndd);
  const float2 nds = make_float2(c.r_k1 * c.scale, c.r_k1 * c.scale);  // -D*scale
#pragma unroll
  for (int ch = 0; ch < CH; ++ch) {
    const int col0 = col_base + 16 * ch;
    uint32_t s[16], a2[16], dp[16], x[16];
    tmem_ld16(acc + 0 * BN + 16 * ch, s);
    tmem_ld16(acc + 1 * BN + 16 * ch, a2);
    if (PASS == 2) {
      tmem_ld16(acc + 2 * BN + 16 * ch, dp);
      tmem_ld16(acc + 3 * BN + 16 * ch, x);
    }
    tmem_wait_ld();
#pragma unroll
    for (int j = 0; j < 16; j += 2) {  // two columns per packed fp32 instruction
      const float2 fa2 = f2(a2[j], a2[j + 1]);
      const float2 arg = __ffma2_rn(f2(s[j], s[j + 1]), sl2, nlc);
      float2 pr = make_float2(ex2(arg.x), ex2(arg.y));
      if (MASKED) {
        const int idx = col0 + j;
        pr.x = (idx >= c.lo && idx <= c.hi) ? pr.x : 0.f;
        pr.y = (idx + 1 >= c.lo && idx + 1 <= c.hi) ? pr.y : 0.f;
      }
      if (PASS == 1) {
        rowacc = __ffma2_rn(pr, fa2, rowacc);
      } else if (FUSED) {
        const float2 q = __fmul2_rn(pr, fa2);
        r[0] = __fadd2_rn(r[0], q);
        r[1] = __ffma2_rn(pr, f2(x[j], x[j + 1]), r[1]);
        r[2] = __ffma2_rn(f2(dp[j], dp[j + 1]), q, r[2]);
        if (FUSED == 2) r[3] = __ffma2_rn(pr, f2(dp[j], dp[j + 1]), r[3]);
      } else {
        const float2 tt = __ffma2_rn(fa2, scale, ndd);
        float2 u = __ffma2_rn(f2(dp[j], dp[j + 1]), tt, f2(x[j], x[j + 1]));
        u = __ffma2_rn(nds, fa2, u);
        rowacc = __ffma2_rn(pr, u, rowacc);
      }
    }
  }
}

// fp32 problems on the tensor cores (SPLIT): every fp32 operand x travels as two bf16 numbers,
// hi = bf16(x) and lo = bf16(x - hi), and a contraction becomes three kind::f16 products with fp32
// accumulation, hi.hi + hi.lo + lo.hi (the lo.lo term, 2^-16 of the result, is dropped).  A row of
// a split tensor in memory is [hi(64) | lo(64)], which is exactly the two 64-column boxes of a
// 128-wide tile, so tile shapes, shared-memory layout and the TMEM budget are those of head dim
// 128; the head dim itself is 64.  The 16-bit tiles the elementwise warps hand back (P, ddP, dS,
// dS2) are split the same way: a thread's 32 fp32 columns of an accumulator take 16 packed columns
// of hi values followed by 16 of lo values.
__device__ __forceinline__ void split_pack(float x, float y, uint32_t& hi, uint32_t& lo) {
  hi = pack_bf16(x, y);
  lo = pack_bf16(x - __uint_as_float(hi << 16), y - __uint_as_float(hi & 0xffff0000u));
}

// D (+)= A . B^T for split operands: boxes (hi, hi), (hi, lo), (lo, hi), four K = 16 steps each.
template <int A_BOX, int B_BOX>
__device__ __forceinline__ void gemm_ss_split(bool leader, uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                              uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int term = 0; term < 3; ++term) {
    const int ab = term == 2 ? 1 : 0, bb = term == 1 ? 1 : 0;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const uint32_t a = a_lo + ((ab * A_BOX + ks * 32) >> 4);
      const uint32_t b = b_lo + ((bb * B_BOX + ks * 32) >> 4);
      umma_ss_split(d_tmem, a, b, kDescHi, idesc, (accumulate || term > 0 || ks > 0) ? 1u : 0u, leader);
    }
  }
}

// Passes 3 and 4 work on a thread's 32 columns of a 64-row streamed tile at once, two columns
// per packed fp32 instruction (fma/mul/add .f32x2).
// First half of a tile: S, A2 -> P = exp2(S*sl2 + nlc), t = scale*A2 - dd; writes ddP = P t (and P
// in pass 3) as bf16 over the accumulators and keeps P and t in registers for the second half.
// In pass 3 the half starts when only S is complete ([S | Q.ddK^T] finished, ddQ.K^T still running
// on the tensor pipe): the exponentials, which the special-function unit bounds, overlap that
// product; `a2_full` is waited for half-way through them and A2 is loaded behind the rest
// (measured: pass 3 3-4 % faster; pass 4, which is at the register limit, up to 8 % slower).
__host__ __device__ constexpr bool early_s(int pass) { return FHOB_EARLY_S && pass == 3; }

template <int PASS, bool MASKED, bool F16, bool SPLIT, class B>
__device__ __forceinline__ bool ew_half_a(uint32_t acc, int col_base, int col_in_tile, const EwCtx& c,
                                          float2 (&ps)[16], float2 (&tt)[16], uint64_t* a2_full, uint32_t parity,
                                          B* bars, int* status) {
  constexpr bool kQStat = PASS != 4;
  constexpr bool kEarlyS = early_s(PASS);
  constexpr int BN = 64;
  uint32_t s[32], a2[32];
  tmem_ld32(acc + 0 * BN, s);
  if (!kEarlyS) tmem_ld32(acc + 1 * BN, a2);
  tmem_wait_ld();
  uint32_t w_ddp[16], w_p[16], w_ddp_lo[16], w_p_lo[16];
  const float2 sl2 = make_float2(c.sl2, c.sl2), scale = make_float2(c.scale, c.scale);
  auto exps = [&](int j4) {
    float c_nlc[4];
    if (kQStat) {
#pragma unroll
      for (int e = 0; e < 4; ++e) c_nlc[e] = c.r_nlc;
    } else {
      load4(c.sv + (0 * BN + col_in_tile + 4 * j4) * 4, c_nlc);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int j = 4 * j4 + 2 * h;  // columns j, j+1
      const float2 arg = __ffma2_rn(f2(s[j], s[j + 1]), sl2, make_float2(c_nlc[2 * h], c_nlc[2 * h + 1]));
      float2 pr = make_float2(ex2(arg.x), ex2(arg.y));
      if (MASKED) {
        const int idx = col_base + j;
        pr.x = (idx >= c.lo && idx <= c.hi) ? pr.x : 0.f;
        pr.y = (idx + 1 >= c.lo && idx + 1 <= c.hi) ? pr.y : 0.f;
      }
      ps[j / 2] = pr;
    }
  };
#pragma unroll
  for (int j4 = 0; j4 < 4; ++j4) exps(j4);
  if (kEarlyS) {
    if (!__all_sync(0xffffffffu, wait_bar(a2_full, parity, bars, status))) return false;
    tc_fence_after();
    tmem_ld32(acc + 1 * BN, a2);
  }
#pragma unroll
  for (int j4 = 4; j4 < 8; ++j4) exps(j4);
  if (kEarlyS) tmem_wait_ld();
#pragma unroll
  for (int j4 = 0; j4 < 8; ++j4) {
    float c_ndd[4];
    if (kQStat) {
#pragma unroll
      for (int e = 0; e < 4; ++e) c_ndd[e] = c.r_ndd;
    } else {
      load4(c.sv + (1 * BN + col_in_tile + 4 * j4) * 4, c_ndd);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int j = 4 * j4 + 2 * h;
      float2 t = __ffma2_rn(f2(a2[j], a2[j + 1]), scale, make_float2(c_ndd[2 * h], c_ndd[2 * h + 1]));
      if (MASKED) {
        const int idx = col_base + j;
        t.x = (idx >= c.lo && idx <= c.hi) ? t.x : 0.f;
        t.y = (idx + 1 >= c.lo && idx + 1 <= c.hi) ? t.y : 0.f;
      }
      const float2 pr = ps[j / 2];
      const float2 ddp = __fmul2_rn(pr, t);
      tt[j / 2] = t;
      if constexpr (SPLIT) {
        split_pack(ddp.x, ddp.y, w_ddp[j / 2], w_ddp_lo[j / 2]);
        if (PASS == 3) split_pack(pr.x, pr.y, w_p[j / 2], w_p_lo[j / 2]);
      } else {
        w_ddp[j / 2] = pack16<F16>(ddp.x, ddp.y);
        if (PASS == 3) w_p[j / 2] = pack16<F16>(pr.x, pr.y);
      }
    }
  }
  // the 16-bit tiles overwrite accumulator columns this thread has already consumed
  tmem_st16(acc + 1 * BN, w_ddp);
  if (PASS == 3) tmem_st16(acc + 0 * BN, w_p);
  if constexpr (SPLIT) {
    tmem_st16(acc + 1 * BN + 16, w_ddp_lo);
    if (PASS == 3) tmem_st16(acc + 0 * BN + 16, w_p_lo);
  }
  return true;
}

// Second half: dP' = dP - D, X' = X - D*dd - b; writes P dP' and P (dP' t + X'), i.e. dS/scale and
// dS2/scale: the factor `scale` is applied once to the finished dQ2 / dK2 accumulator instead.
template <int PASS, bool MASKED, bool F16, bool SPLIT>
__device__ __forceinline__ void ew_half_b(uint32_t acc, int col_base, int col_in_tile, const EwCtx& c,
                                          const float2 (&ps)[16], const float2 (&tt)[16]) {
  constexpr bool kQStat = PASS != 4;
  constexpr int BN = 64;
  uint32_t dp[32], x[32];
  tmem_ld32(acc + 2 * BN, dp);
  tmem_ld32(acc + 3 * BN, x);
  tmem_wait_ld();
  uint32_t w_ds[16], w_ds2[16], w_ds_lo[16], w_ds2_lo[16];
#pragma unroll
  for (int j4 = 0; j4 < 8; ++j4) {
    float c_k1[4], c_k23[4];
    if (kQStat) {
#pragma unroll
      for (int e = 0; e < 4; ++e) { c_k1[e] = c.r_k1; c_k23[e] = c.r_k23; }
    } else {
      load4(c.sv + (2 * BN + col_in_tile + 4 * j4) * 4, c_k1);
      load4(c.sv + (3 * BN + col_in_tile + 4 * j4) * 4, c_k23);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int j = 4 * j4 + 2 * h;
      const float2 dpp = __fadd2_rn(f2(dp[j], dp[j + 1]), make_float2(c_k1[2 * h], c_k1[2 * h + 1]));
      const float2 xp = __fadd2_rn(f2(x[j], x[j + 1]), make_float2(c_k23[2 * h], c_k23[2 * h + 1]));
      const float2 u = __ffma2_rn(dpp, tt[j / 2], xp);
      float2 ds = __fmul2_rn(ps[j / 2], dpp);
      float2 ds2 = __fmul2_rn(ps[j / 2], u);
      if (MASKED) {
        const int idx = col_base + j;
        const bool ok0 = idx >= c.lo && idx <= c.hi, ok1 = idx + 1 >= c.lo && idx + 1 <= c.hi;
        ds.x = ok0 ? ds.x : 0.f;   ds.y = ok1 ? ds.y : 0.f;
        ds2.x = ok0 ? ds2.x : 0.f; ds2.y = ok1 ? ds2.y : 0.f;
      }
      if constexpr (SPLIT) {
        split_pack(ds.x, ds.y, w_ds[j / 2], w_ds_lo[j / 2]);
        split_pack(ds2.x, ds2.y, w_ds2[j / 2], w_ds2_lo[j / 2]);
      } else {
        w_ds[j / 2] = pack16<F16>(ds.x, ds.y);
        w_ds2[j / 2] = pack16<F16>(ds2.x, ds2.y);
      }
    }
  }
  tmem_st16(acc + 2 * BN, w_ds);
  tmem_st16(acc + 3 * BN, w_ds2);
  if constexpr (SPLIT) {
    tmem_st16(acc + 2 * BN + 16, w_ds_lo);
    tmem_st16(acc + 3 * BN + 16, w_ds2_lo);
  }
}

template <int PASS, int DQK, int DV, int BN, int FUSED = 0, bool F16 = false, bool SPLIT = false>
__global__ void __launch_bounds__(NTHREADS, 1) tc_pass_kernel(const __grid_constant__ TcParams p) {
  static_assert(FUSED == 0 || PASS == 2, "only pass 2 has a fused form");
  static_assert(!SPLIT || (DQK == 128 && DV == 128 && !F16), "split fp32 operands are [hi(64) | lo(64)] bf16 rows");
  using C = Cfg<PASS, DQK, DV, BN>;
  constexpr bool kQStat = PASS != 4;
  // passes 1, 2: a third warp issues the second product of group A (their tensor pipe has the room;
  // in passes 3, 4 the extra issuer only delayed group A)
  constexpr bool kThirdIssuer = PASS <= 2;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* stat_tiles = smem;
  uint8_t* strm_tiles = smem + C::STAT_BYTES;
  Bars* bars = reinterpret_cast<Bars*>(strm_tiles + C::NSLOT * C::SLOT_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x / p.tiles_per_head;
  const int tile_in_head = blockIdx.x - head * p.tiles_per_head;
  // causal: longest tiles first (late queries in passes 1-3, early keys in pass 4)
  const int tile = kQStat ? p.tiles_per_head - 1 - tile_in_head : tile_in_head;
  const int m0 = tile * BM;
  const int n_stat = kQStat ? p.n_q : p.n_k;
  const int n_strm = kQStat ? p.n_k : p.n_q;
  const int off = p.n_k - p.n_q;

  int t_begin, t_end;
  visible_tiles(kQStat, m0, BM, BN, n_strm, off, p.causal, p.window, t_begin, t_end);
  const int n_iter = t_end - t_begin;

  // ---- set-up
  if (threadIdx.x == 0) {
    if (smem_u32(smem) & 1023u) atomicOr(p.status, FHOB_ERR_SMEM_ALIGN);
    mbar_init(&bars->stat_full, 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&bars->strm_full[i], 1);
      mbar_init(&bars->strm_free[i], PASS == 1 ? 2 : (PASS == 2 ? 3 : 2));  // one commit per issuing warp
    }
    for (int i = 0; i < 2; ++i) {
      // commits per phase: in passes 1, 2 group A comes from two warps; pass 2 adds group B to the stage
      mbar_init(&bars->s_full[i], PASS == 1 ? 2 : (PASS == 2 ? 3 : 1));
      mbar_init(&bars->s_free[i], EW_THREADS);
      mbar_init(&bars->p_full[i], EW_THREADS);
    }
    mbar_init(&bars->out_full, 2);
    mbar_init(&bars->chain_go, 1);
    mbar_init(&bars->s_ready, 1);
    mbar_init(&bars->a2_go, 1);
    mbar_init(&bars->teardown[2], 1);
    mbar_init(&bars->teardown[0], 1);
    mbar_init(&bars->teardown[1], 1);
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
  // The CTA allocates all 512 columns, so the allocation starts at lane 0, column 0.  Using the
  // constant keeps every TMEM address of the MMA issue loop an immediate; a different answer from
  // the allocator is reported through the status word.
  constexpr uint32_t tmem_base = 0;
  if (threadIdx.x == 0 && *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base) != 0)
    atomicOr(p.status, FHOB_ERR_TMEM_BASE);

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
        if (!wait_bar(&bars->strm_free[slot], ((it / C::NSLOT) & 1) ^ 1, bars, p.status)) break;
        mbar_arrive_expect_tx(&bars->strm_full[slot], C::SLOT_BYTES);
        uint8_t* dst = strm_tiles + slot * C::SLOT_BYTES;
        const int n0 = (t_begin + it) * BN;
#pragma unroll
        for (int i = 0; i < C::NSTRM; ++i)
          for (int bx = 0; bx < C::tile_d(i) / 64; ++bx)
            tma_load_4d(dst + C::strm_base(i) + bx * C::strm_box(i), &p.strm[i], &bars->strm_full[slot], bx * 64,
                        n0, head_h, head_b);
        if (PASS == 4) {
          const size_t vo = static_cast<size_t>(head) * row_stride(p.n_q) + n0;
          uint8_t* sv = dst + C::STRM_BYTES;
          bulk_load(sv + 0 * BN * 4, p.nlc + vo, BN * 4, &bars->strm_full[slot]);
          bulk_load(sv + 1 * BN * 4, p.ndd + vo, BN * 4, &bars->strm_full[slot]);
          bulk_load(sv + 2 * BN * 4, p.k1 + vo, BN * 4, &bars->strm_full[slot]);
          bulk_load(sv + 3 * BN * 4, p.k23 + vo, BN * 4, &bars->strm_full[slot]);
        }
        issued = it + 1;
      }
      // drain: every load issued above must have landed before the CTA may exit
      wait_bar(&bars->stat_full, 0, bars, p.status);
      for (int it = issued > C::NSLOT ? issued - C::NSLOT : 0; it < issued; ++it) {
        const int slot = it % C::NSLOT;
        const long long start = clock64();
        while (!mbar_try_wait(&bars->strm_full[slot], (it / C::NSLOT) & 1)) {
          if (clock64() - start > kTimeoutCycles) {
            atomicOr(p.status, FHOB_ERR_TIMEOUT);
            break;
          }
        }
      }
    }
  } else if (warp == MMA_WARP || warp == MMA_WARP2) {
    // ================================================= MMA issuers
    // The whole warp runs the loop so that addresses and descriptors stay warp-uniform; one lane
    // issues the MMAs and commits.  chain 0 = group A side, chain 1 = group B side.
    const int chain = warp == MMA_WARP ? 0 : 1;
    const bool has_work = n_iter > 0 && (chain == 0 || PASS >= 2);
    if (has_work) {
      const bool leader = lane == 0;
      auto wait_all = [&](uint64_t* bar, uint32_t parity) {
        return __all_sync(0xffffffffu, wait_bar(bar, parity, bars, p.status)) != 0;
      };
      auto commit = [&](uint64_t* bar) {
        if (leader) umma_commit(bar);
      };
      constexpr uint32_t idesc_s1 = umma_idesc_bf16(BM, BN, false, false, F16);      // one streamed tile
      constexpr uint32_t idesc_s2 = umma_idesc_bf16(BM, 2 * BN, false, false, F16);  // a stacked pair
      constexpr uint32_t idesc_o0 = umma_idesc_bf16(BM, DQK, false, true, F16);  // dQ2 | dK2
      constexpr uint32_t idesc_o1 = umma_idesc_bf16(BM, DV, false, true, F16);   // ddO | dV2
      constexpr uint32_t idesc_o64 = umma_idesc_bf16(BM, 64, false, true, F16);  // split operands: the hi box alone
      constexpr int kStatBox = BM * 128;
      // low descriptor words of the tiles: K-major use (LBO field unused, set to 1) and MN-major
      // use of streamed tile i (LBO = distance between its two 64-column boxes)
      const uint32_t stat_lo = umma_desc_lo(smem_u32(stat_tiles), 16);
      const uint32_t strm_lo = umma_desc_lo(smem_u32(strm_tiles), 16);
      constexpr uint32_t kSlot16 = C::SLOT_BYTES >> 4;
      auto stat_i = [&](int i) { return stat_lo + (C::stat_off(i) >> 4); };
      auto k_lo = [&](uint32_t slot_lo, int i) { return slot_lo + (C::strm_base(i) >> 4); };
      auto mn_lo = [&](uint32_t slot_lo, int i) {
        return slot_lo - (1u << 16) + (C::strm_base(i) >> 4) + (static_cast<uint32_t>(C::strm_box(i) >> 4) << 16);
      };
      bool ok = wait_all(&bars->stat_full, 0);
      // one score-shaped product: contraction over KD columns, or over hi/lo boxes for split operands
      auto scores = [&](auto kd, auto b_box, uint32_t d, uint32_t a, uint32_t b, uint32_t idesc, bool accumulate) {
        if constexpr (SPLIT) gemm_ss_split<kStatBox, decltype(b_box)::value>(leader, d, a, b, idesc, accumulate);
        else gemm_ss<decltype(kd)::value, kStatBox, decltype(b_box)::value>(leader, d, a, b, idesc, accumulate);
      };
      using KQ = std::integral_constant<int, DQK>;
      using KV = std::integral_constant<int, DV>;
      using Box0 = std::integral_constant<int, C::strm_box(0)>;
      using Box2 = std::integral_constant<int, C::strm_box(2)>;

      // score-shaped products of this chain for tile `it` (waits for the tile's shared-memory slot)
      //   chain 0, group A: [S | stat0.strm1^T] as one N = 2*BN product, then A2 += stat1.strm0^T
      //   chain 1, group B: [dP | X] (one stacked product in passes 2, 3; two products in pass 4)
      auto issue_scores = [&](int it, uint32_t acc) -> bool {
        const int slot = it % C::NSLOT;
        if (!wait_all(&bars->strm_full[slot], (it / C::NSLOT) & 1)) return false;
        tc_fence_after();
        const uint32_t sl = strm_lo + slot * kSlot16;
        if (chain == 0) {
          scores(KQ{}, Box0{}, acc, stat_lo, k_lo(sl, 0), idesc_s2, false);
          if (kThirdIssuer) {
            // A2 += stat1 . strm0^T is issued by the third warp, strictly behind the stacked product
            // so that the order of the fp32 accumulation (and with it every result bit) is fixed
            if (leader) mbar_arrive(&bars->a2_go);
          } else {
            if (early_s(PASS)) commit(&bars->s_ready);
            scores(KQ{}, Box0{}, acc + BN, stat_i(1), k_lo(sl, 0), idesc_s1, true);
          }
        } else if (PASS == 4) {
          scores(KV{}, Box2{}, acc + 2 * BN, stat_i(2), k_lo(sl, 2), idesc_s1, false);
          scores(KV{}, Box2{}, acc + 3 * BN, stat_i(3), k_lo(sl, 2), idesc_s1, false);
        } else {
          scores(KV{}, Box2{}, acc + 2 * BN, stat_i(2), k_lo(sl, 2), idesc_s2, false);
        }
        return true;
      };

      if (PASS <= 2) {
        for (int it = 0; ok && it < n_iter; ++it) {
          const int stage = it % C::NSS;
          const uint32_t acc = tmem_base + C::OUT_COLS + stage * C::STAGE_COLS;
          ok = wait_all(&bars->s_free[stage], ((it / C::NSS) & 1) ^ 1);
          ok = ok && issue_scores(it, acc);
          if (!ok) break;
          commit(&bars->s_full[stage]);
          commit(&bars->strm_free[it % C::NSLOT]);
        }
      } else {
        // One TMEM stage, pipelined per chain: scores(t) -> [elementwise half] -> outputs(t) ->
        // scores(t+1) ...  The bf16 tiles sit where the chain's own accumulators were, and its
        // MMAs execute in issue order, so scores(t+1) cannot overtake outputs(t).
        const uint32_t acc = tmem_base + C::OUT_COLS;
        const uint32_t out0 = tmem_base, out1 = tmem_base + C::OUT0_COLS;
        ok = ok && issue_scores(0, acc);
        if (ok) commit(&bars->s_full[chain]);
        for (int it = 0; ok && it < n_iter; ++it) {
          const uint32_t sl = strm_lo + (it % C::NSLOT) * kSlot16;
          const bool accum = it > 0;
          ok = wait_all(&bars->p_full[chain], it & 1);
          if (!ok) break;
          tc_fence_after();
          // one output product, A = 16-bit tile in TMEM; split operands: A_hi . [B_hi | B_lo] fills
          // both 64-column halves of the accumulator (they are added in the epilogue), then
          // A_lo . B_hi goes on top of the first half
          auto outputs = [&](uint32_t out, uint32_t a_region, uint32_t b, uint32_t idesc, bool accumulate) {
            gemm_ts<BN>(leader, out, a_region, b, idesc, accumulate);
            if constexpr (SPLIT) gemm_ts<BN>(leader, out, a_region + 16, b, idesc_o64, true);
          };
          if (chain == 0) {
            outputs(out1, acc + 1 * BN, mn_lo(sl, 2), idesc_o1, accum);              // ddP . V | dO
            if (kQStat) outputs(out1, acc + 0 * BN, mn_lo(sl, 3), idesc_o1, true);   // P . ddV
          } else {
            outputs(out0, acc + 2 * BN, mn_lo(sl, 1), idesc_o0, accum);  // dS  . ddK | ddQ
            outputs(out0, acc + 3 * BN, mn_lo(sl, 0), idesc_o0, true);   // dS2 . K   | Q
          }
          commit(&bars->strm_free[it % C::NSLOT]);
          // Chain 1's group A of the next tile gates the next elementwise half, while chain 2's
          // group B is needed half a tile later: chain 2 lets chain 1 issue first, so the tensor
          // pipe runs them in that order.
          if (chain == 1) {
            ok = wait_all(&bars->chain_go, it & 1);
            if (!ok) break;
          }
          if (it + 1 < n_iter) {
            ok = issue_scores(it + 1, acc);
            if (!ok) break;
            commit(&bars->s_full[chain]);
          }
          if (chain == 0 && leader) mbar_arrive(&bars->chain_go);
        }
      }
      if (ok) {
        if (PASS >= 3) commit(&bars->out_full);
      } else {
        // abort path: no tcgen05.mma may still be reading shared memory or TMEM at exit
        commit(&bars->teardown[chain]);
        const long long start = clock64();
        while (!mbar_try_wait(&bars->teardown[chain], 0)) {
          if (clock64() - start > kTimeoutCycles) break;
        }
      }
    }
  } else if (warp == MMA_WARP3) {
    // ================================================= third issuer: A2 += stat1 . strm0^T
    if (kThirdIssuer && n_iter > 0) {
      const bool leader = lane == 0;
      auto wait_all = [&](uint64_t* bar, uint32_t parity) {
        return __all_sync(0xffffffffu, wait_bar(bar, parity, bars, p.status)) != 0;
      };
      constexpr uint32_t idesc_s1 = umma_idesc_bf16(BM, BN, false, false, F16);
      constexpr int kStatBox = BM * 128;
      const uint32_t stat_lo = umma_desc_lo(smem_u32(stat_tiles), 16);
      const uint32_t strm_lo = umma_desc_lo(smem_u32(strm_tiles), 16);
      constexpr uint32_t kSlot16 = C::SLOT_BYTES >> 4;
      bool ok = wait_all(&bars->stat_full, 0);
      for (int it = 0; ok && it < n_iter; ++it) {
        const int slot = it % C::NSLOT;
        const int stage = PASS <= 2 ? it % C::NSS : 0;
        // chain 1 has waited for the stage and issued [S | stat0.strm1^T], which zero-initialises A2
        ok = wait_all(&bars->a2_go, it & 1) && wait_all(&bars->strm_full[slot], (it / C::NSLOT) & 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = tmem_base + C::OUT_COLS + (PASS <= 2 ? stage * C::STAGE_COLS : 0);
        if constexpr (SPLIT)
          gemm_ss_split<kStatBox, C::strm_box(0)>(leader, acc + BN, stat_lo + (C::stat_off(1) >> 4),
                                                  strm_lo + slot * kSlot16 + (C::strm_base(0) >> 4), idesc_s1, true);
        else
          gemm_ss<DQK, kStatBox, C::strm_box(0)>(leader, acc + BN, stat_lo + (C::stat_off(1) >> 4),
                                                 strm_lo + slot * kSlot16 + (C::strm_base(0) >> 4), idesc_s1, true);
        if (leader) {
          umma_commit(&bars->s_full[stage]);
          umma_commit(&bars->strm_free[slot]);
        }
      }
      if (!ok && leader) {
        umma_commit(&bars->teardown[2]);
        const long long start = clock64();
        while (!mbar_try_wait(&bars->teardown[2], 0)) {
          if (clock64() - start > kTimeoutCycles) break;
        }
      }
    }
  } else {
    // ================================================= elementwise warps
    const int quad = warp & 3, half = (warp - EW_WARP0) >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int g_row = m0 + row;  // stationary row of this thread
    const size_t vec_head = static_cast<size_t>(head) * row_stride(p.n_q);
    EwCtx c;
    c.scale = p.scale;
    c.sl2 = p.scale * kLog2e;
    c.r_nlc = c.r_k1 = c.r_ndd = c.r_k23 = 0.f;
    if (kQStat && g_row < p.n_q) {
      c.r_nlc = p.nlc[vec_head + g_row];
      if (PASS >= 2) {
        if (FUSED != 2) c.r_k1 = p.k1[vec_head + g_row];
        if (FUSED == 0) c.r_ndd = p.ndd[vec_head + g_row];
      }
      if (PASS >= 3) c.r_k23 = p.k23[vec_head + g_row];
    }
    c.sv = 0;
    if (kQStat) {
      c.lo = 0;
      c.hi = p.n_k - 1;
      if (p.causal && g_row + off < c.hi) c.hi = g_row + off;
      if (p.window > 0 && g_row + off - p.window + 1 > 0) c.lo = g_row + off - p.window + 1;
    } else {
      c.lo = p.causal ? g_row - off : 0;
      if (c.lo < 0) c.lo = 0;
      c.hi = p.n_q - 1;
      if (p.window > 0 && g_row - off + p.window - 1 < c.hi) c.hi = g_row - off + p.window - 1;
    }
    float2 racc[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
    float2& rowacc = racc[0];
    bool ok = true;

    for (int it = 0; it < n_iter; ++it) {
      const int n0 = (t_begin + it) * BN;
      // does any element of this tile need masking?  (CTA-uniform: depends on tile coordinates only)
      bool masked = n0 + BN > n_strm;
      if (p.causal) {
        if (kQStat) masked = masked || (n0 + BN - 1 > m0 + off);
        else masked = masked || (n0 + off < m0 + BM - 1);
        if (p.window > 0) {
          // the pair of the tile that is furthest apart: last query row against first key row
          if (kQStat) masked = masked || (m0 + BM - 1 + off - n0 >= p.window);
          else masked = masked || (n0 + BN - 1 + off - m0 >= p.window);
        }
      }
      const int col_base = n0 + half * (BN / 2);
      if constexpr (PASS <= 2) {
        const int stage = it % C::NSS;
        ok = __all_sync(0xffffffffu, wait_bar(&bars->s_full[stage], (it / C::NSS) & 1, bars, p.status));
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = tmem_base + lane_base + stage * C::STAGE_COLS + half * (BN / 2);
        if (masked) ew_reduce<PASS, BN, true, FUSED>(acc, col_base, c, racc);
        else ew_reduce<PASS, BN, false, FUSED>(acc, col_base, c, racc);
        tc_fence_before();
        mbar_arrive(&bars->s_free[stage]);
      } else {
        const uint32_t acc = tmem_base + lane_base + C::OUT_COLS + half * (BN / 2);
        float2 ps[16], tt[16];
        if (PASS == 4) {
          // the slot's constants were written by the TMA unit: observe its barrier before reading them
          const int slot = it % C::NSLOT;
          ok = __all_sync(0xffffffffu, wait_bar(&bars->strm_full[slot], (it / C::NSLOT) & 1, bars, p.status));
          if (!ok) break;
          c.sv = smem_u32(strm_tiles + slot * C::SLOT_BYTES + C::STRM_BYTES);
        }
        ok = __all_sync(0xffffffffu, wait_bar(early_s(PASS) ? &bars->s_ready : &bars->s_full[0], it & 1, bars, p.status));
        if (!ok) break;
        tc_fence_after();
        if (masked) ok = ew_half_a<PASS, true, F16, SPLIT>(acc, col_base, half * (BN / 2), c, ps, tt, &bars->s_full[0], it & 1, bars, p.status);
        else ok = ew_half_a<PASS, false, F16, SPLIT>(acc, col_base, half * (BN / 2), c, ps, tt, &bars->s_full[0], it & 1, bars, p.status);
        if (!ok) break;
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&bars->p_full[0]);
        ok = __all_sync(0xffffffffu, wait_bar(&bars->s_full[1], it & 1, bars, p.status));
        if (!ok) break;
        tc_fence_after();
        if (masked) ew_half_b<PASS, true, F16, SPLIT>(acc, col_base, half * (BN / 2), c, ps, tt);
        else ew_half_b<PASS, false, F16, SPLIT>(acc, col_base, half * (BN / 2), c, ps, tt);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&bars->p_full[1]);
      }
    }

    // ---- results
    if (FUSED) {
      // dd = scale * sum P A2;  b = sum P X + scale * sum dP P A2 - 2 D dd, because sum P dP = D
      float r1 = racc[0].x + racc[0].y;
      float rb = (racc[1].x + racc[1].y) + c.scale * (racc[2].x + racc[2].y);
      if (half == 1) bars->red[row] = r1;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (half == 0) r1 += bars->red[row];
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (half == 1) bars->red[row] = rb;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (half == 0) rb += bars->red[row];
      float d_row = -c.r_k1;
      if (FUSED == 2) {
        // D = sum P dP (the caller passed no O): it is also what passes 3 and 4 read as k1 = -D
        d_row = racc[3].x + racc[3].y;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (half == 1) bars->red[row] = d_row;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (half == 0) d_row += bars->red[row];
      }
      if (half == 0 && ok && g_row < p.n_q) {
        const float dd = c.scale * r1;
        p.ndd[vec_head + g_row] = -dd;
        p.k23[vec_head + g_row] = d_row * dd - rb;  // -D*dd - b = D*dd - (sum P X + scale * sum dP P A2)
        if (FUSED == 2) const_cast<float*>(p.k1)[vec_head + g_row] = -d_row;
      }
    } else if (PASS <= 2) {
      if (half == 1) bars->red[row] = rowacc.x + rowacc.y;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (half == 0 && ok && g_row < p.n_q) {
        const float tot = rowacc.x + rowacc.y + bars->red[row];
        if (PASS == 1) p.ndd[vec_head + g_row] = -c.scale * tot;     // -dd, dd = scale * sum P A2
        else p.k23[vec_head + g_row] = -c.r_k1 * c.r_ndd - tot;      // -D*dd - b, b = sum P dP2
      }
    } else {
      if (n_iter > 0) ok = ok && __all_sync(0xffffffffu, wait_bar(&bars->out_full, 0, bars, p.status));
      tc_fence_after();
      if (ok) {
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
        // split operands: a result has 64 fp32 columns, the sum of the two 64-column halves of its accumulator
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
        // dS and dS2 were stored without the factor `scale`: it is applied to dQ2 | dK2 here
        if constexpr (SPLIT) {
          store_out_split(p.d_out0, 0, p.out0, c.scale);
          store_out_split(p.d_out1, C::OUT0_COLS, p.out1, 1.f);
        } else {
          store_out(std::integral_constant<int, DQK>{}, p.d_out0, 0, p.out0, c.scale);
          store_out(std::integral_constant<int, DV>{}, p.d_out1, C::OUT0_COLS, p.out1, 1.f);
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

// ------------------------------------------------------------------ host side

// fp32 rows of d <= 64 columns -> [hi(64) | lo(64)] bf16 rows (see split_pack), zero beyond d: one
// thread per pair of columns of the 64-wide row.  One launch converts all the tensors a call needs
// (blockIdx.y = tensor), which matters for the small problems whose time is mostly launches.
struct SplitJobs {
  const float* src[7];
  uint32_t* dst[7];
  long pairs[7];
  int d[7], n_rows[7];
  View view[7];
};
__global__ void split_rows_kernel(const __grid_constant__ SplitJobs jobs) {
  const int t = blockIdx.y;
  const long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= jobs.pairs[t]) return;
  const int d = jobs.d[t], n_rows = jobs.n_rows[t];
  const View& v = jobs.view[t];
  const long row = i >> 5;          // 32 pairs of columns per row of 64; rows of the copy are dense (bh, n, 128)
  const int c2 = static_cast<int>(i & 31);
  const long bh = row / n_rows, r = row - bh * n_rows;
  const float* s = jobs.src[t] + (bh / v.heads) * v.batch + (bh % v.heads) * v.head + r * v.row;   // the source may be a view
  const float2 x = 2 * c2 < d ? *reinterpret_cast<const float2*>(s + 2 * c2) : make_float2(0.f, 0.f);
  uint32_t hi, lo;
  split_pack(x.x, x.y, hi, lo);
  uint32_t* dst = jobs.dst[t];
  dst[row * 64 + c2] = hi;          // a split row is 128 bf16 = 64 words: hi in words [0, 32), lo in [32, 64)
  dst[row * 64 + 32 + c2] = lo;
}

template <int PASS, int DQK, int DV, int BN, int FUSED = 0, bool F16 = false, bool SPLIT = false>
int launch(const FhobProblem& p, cudaStream_t s) {
  using C = Cfg<PASS, DQK, DV, BN>;
  constexpr auto kernel = tc_pass_kernel<PASS, DQK, DV, BN, FUSED, F16, SPLIT>;
  RowVectors rv = row_vectors(p);
  TcParams tp;
  memset(&tp, 0, sizeof(tp));
  const void* q_side[3] = {p.q, p.ddq, p.d_o};
  const void* k_side[4] = {p.k, p.ddk, p.v, p.ddv};
  if (SPLIT) {
    // the kernels read the bf16 hi/lo copies the preparation step left behind the row vectors
    SplitBuffers sb = split_buffers(p);
    q_side[0] = sb.q; q_side[1] = sb.ddq; q_side[2] = sb.d_o;
    k_side[0] = sb.k; k_side[1] = sb.ddk; k_side[2] = sb.v; k_side[3] = sb.ddv;
  }
  // A head dim below the tile width (any multiple of 8 up to 128) needs nothing but the right
  // tensor map: the 64-column boxes reach past the end of a row, the TMA unit fills those columns
  // with zeros, zeros add nothing to a contraction, and the epilogue stores only the columns that exist.
  const int d_mem[2] = {SPLIT ? 128 : p.d, SPLIT ? 128 : head_dim_v(p)};   // columns in memory of the two tile kinds
  // where each input lives: the caller's layout, or contiguous (always so for the split copies)
  const int q_ids[3] = {kTenQ, kTenDDQ, kTenDO}, k_ids[4] = {kTenK, kTenDDK, kTenV, kTenDDV};
  auto view = [&](int id, int n_rows, int d) {
    return SPLIT ? contiguous_view(p.bh, n_rows, d) : tensor_view(p, id, n_rows, d);
  };
  int st = FHOB_OK;
  if (PASS != 4) {
    for (int i = 0; i < C::NSTAT && st == FHOB_OK; ++i)
      st = make_map(&tp.stat[i], q_side[i], view(q_ids[i], p.n_q, d_mem[i < 2 ? 0 : 1]), p.n_q, d_mem[i < 2 ? 0 : 1], BM, F16);
    for (int i = 0; i < C::NSTRM && st == FHOB_OK; ++i)
      st = make_map(&tp.strm[i], k_side[i], view(k_ids[i], p.n_k, d_mem[i < 2 ? 0 : 1]), p.n_k, d_mem[i < 2 ? 0 : 1], BN, F16);
  } else {
    for (int i = 0; i < C::NSTAT && st == FHOB_OK; ++i)
      st = make_map(&tp.stat[i], k_side[i], view(k_ids[i], p.n_k, d_mem[i < 2 ? 0 : 1]), p.n_k, d_mem[i < 2 ? 0 : 1], BM, F16);
    for (int i = 0; i < C::NSTRM && st == FHOB_OK; ++i)
      st = make_map(&tp.strm[i], q_side[i], view(q_ids[i], p.n_q, d_mem[i < 2 ? 0 : 1]), p.n_q, d_mem[i < 2 ? 0 : 1], BN, F16);
  }
  if (st != FHOB_OK) return st;
  tp.heads = (!SPLIT && p.layout) ? p.layout->heads : p.bh;
  tp.d_out0 = p.d;               // columns of the results in memory (split operands: up to 64 fp32 columns)
  tp.d_out1 = head_dim_v(p);
  tp.nlc = rv.nlc; tp.k1 = rv.k1; tp.ndd = rv.ndd; tp.k23 = rv.k23;
  tp.out0 = static_cast<uint16_t*>(PASS == 3 ? p.dq2 : p.dk2);
  tp.out1 = static_cast<uint16_t*>(PASS == 3 ? p.ddo : p.dv2);
  tp.status = rv.status;
  tp.n_q = p.n_q; tp.n_k = p.n_k; tp.causal = p.causal; tp.window = p.window; tp.scale = p.scale;
  const int n_stat = PASS == 4 ? p.n_k : p.n_q;
  tp.tiles_per_head = (n_stat + BM - 1) / BM;
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

template <int DQK, int DV, bool F16, bool SPLIT = false>
int dispatch(int pass, const FhobProblem& p, cudaStream_t s) {
  switch (pass) {
    // pass 1 streams 128-row tiles (the stacked [K ; ddK] operand reaches N = 256), the others 64;
    // it touches no tile of the second head dim
    case 1: return launch<1, DQK, DQK, 128, 0, F16, SPLIT>(p, s);
    case 2: return launch<2, DQK, DV, 64, 0, F16, SPLIT>(p, s);
    case 12: return launch<2, DQK, DV, 64, 1, F16, SPLIT>(p, s);  // passes 1 and 2 in one sweep
    case 13: return launch<2, DQK, DV, 64, 2, F16, SPLIT>(p, s);  // the same, also producing D = sum P dP (no O given)
    case 3: return launch<3, DQK, DV, 64, 0, F16, SPLIT>(p, s);
    case 4: return launch<4, DQK, DV, 64, 0, F16, SPLIT>(p, s);
  }
  return FHOB_ERR_ARG;
}

template <bool F16>
int dispatch_dims(int pass, const FhobProblem& p, cudaStream_t s) {
  // tile widths: the head dims rounded up to 64 or 128
  const int dv = head_dim_v(p);
  if (p.d <= 64) return dv <= 64 ? dispatch<64, 64, F16>(pass, p, s) : dispatch<64, 128, F16>(pass, p, s);
  return dv <= 64 ? dispatch<128, 64, F16>(pass, p, s) : dispatch<128, 128, F16>(pass, p, s);
}

int check_arch() {
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

}  // namespace

bool tc_supported(const FhobProblem& p) {
  const int dv = head_dim_v(p);
  if (p.dtype == FHOB_F32) return tc_split_supported(p);
  // 16-bit storage: any head dims up to 128 whose rows stay 16-byte aligned
  return (p.dtype == FHOB_BF16 || p.dtype == FHOB_F16) && p.d > 0 && p.d <= 128 && p.d % 8 == 0 && dv <= 128 &&
         dv % 8 == 0;
}

// fp32 problems take the tensor-core path when both head dims are at most 64 (and keep rows 16-byte
// aligned) and the workspace has room for the bf16 hi/lo copies of the seven inputs
// (fhob_workspace_bytes_problem says how much)
bool tc_split_supported(const FhobProblem& p) {
  return split_dims_ok(p) && p.workspace && p.workspace_bytes >= split_workspace_bytes(p);
}

int tc_split_inputs(const FhobProblem& p, cudaStream_t s, int which) {
  if (!tc_split_supported(p)) return FHOB_ERR_SHAPE;
  SplitBuffers sb = split_buffers(p);
  const void* src[7] = {p.q, p.ddq, p.d_o, p.k, p.ddk, p.v, p.ddv};   // bit i of `which` = tensor i
  const int ids[7] = {kTenQ, kTenDDQ, kTenDO, kTenK, kTenDDK, kTenV, kTenDDV};
  void* dst[7] = {sb.q, sb.ddq, sb.d_o, sb.k, sb.ddk, sb.v, sb.ddv};
  SplitJobs jobs;
  int count = 0;
  long most = 0;
  for (int i = 0; i < 7; ++i) {
    if (!(which & (1 << i))) continue;
    if (!src[i]) return FHOB_ERR_ARG;
    const int n_rows = i < 3 ? p.n_q : p.n_k;
    const bool v_side = i == 2 || i >= 5;   // dO, V, ddV
    const int d = v_side ? head_dim_v(p) : p.d;
    jobs.src[count] = static_cast<const float*>(src[i]);
    jobs.dst[count] = static_cast<uint32_t*>(dst[i]);
    jobs.pairs[count] = static_cast<long>(p.bh) * n_rows * 32;
    jobs.d[count] = d;
    jobs.n_rows[count] = n_rows;
    jobs.view[count] = tensor_view(p, ids[i], n_rows, d);
    most = jobs.pairs[count] > most ? jobs.pairs[count] : most;
    ++count;
  }
  if (count == 0) return FHOB_OK;
  for (int i = count; i < 7; ++i) {   // unused entries: defined, never read
    jobs.src[i] = nullptr; jobs.dst[i] = nullptr; jobs.pairs[i] = 0; jobs.d[i] = 0; jobs.n_rows[i] = 1;
    jobs.view[i] = jobs.view[0];
  }
  const long blocks = (most + 255) / 256;
  if (blocks > 0x7fffffffL) return FHOB_ERR_SHAPE;
  split_rows_kernel<<<dim3(static_cast<unsigned>(blocks), count), 256, 0, s>>>(jobs);
  FHOB_CUDA_OK(cudaGetLastError());
  return FHOB_OK;
}

int tc_pass(int pass, const FhobProblem& p, cudaStream_t s) {
  if (!tc_supported(p)) return FHOB_ERR_SHAPE;
  int st = check_arch();
  if (st != FHOB_OK) return st;
  if (p.dtype == FHOB_F32) return dispatch<128, 128, false, true>(pass, p, s);
  return p.dtype == FHOB_F16 ? dispatch_dims<true>(pass, p, s) : dispatch_dims<false>(pass, p, s);
}

}  // namespace fhob
