// Tensor-core kernels of the double-backward attention operator for sm_100a:
// TMA tile loads -> tcgen05.mma with fp32 accumulators in TMEM -> tcgen05.ld
// into registers for the elementwise math -> (passes 3, 4) bf16 tiles written
// back to TMEM and used as the A operand of the output products.
//
// One kernel template covers the four passes (reference: passes 1-3 are the
// three key loops of bwdbwd_kernel_stage1, fhog/triton_bwdbwd.py:178-313;
// pass 4 is bwdbwd_kernel_stage2, :321-535).  A CTA owns BM = 128 "stationary"
// rows of one head (queries in passes 1-3, keys in pass 4) which become the 128
// TMEM lanes, and streams BN-row tiles of the other side:
//
//   score-shaped accumulators (128 x BN fp32 each, K-major smem x K-major smem):
//     S  = stat0 . strm0^T          A2 = stat1 . strm0^T + stat0 . strm1^T
//     dP = stat2 . strm2^T          X  = stat2 . strm3^T            (pass 4: X = stat3 . strm2^T)
//   output accumulators (128 x D fp32 each, A = bf16 tile in TMEM, B = streamed tile read MN-major):
//     pass 3: dQ2 += dS . ddK + dS2 . K       ddO += ddP . V + P . ddV
//     pass 4: dK2 += dS^T . ddQ + dS2^T . Q   dV2 += ddP^T . dO
//
// Warp roles (320 threads): warps 0-7 elementwise (warp w owns TMEM lanes
// 32*(w%4).., column half w/4), warp 8 = TMA producer (one lane), warp 9 =
// MMA issuer (one lane) and TMEM allocator.  Every mbarrier wait is bounded:
// when it runs out the CTA raises the status word, drains and exits.
#include <cuda.h>

#include <cstdio>
#include <cstring>

#include "fhob_common.cuh"
#include "sm100_ptx.cuh"

namespace fhob {
namespace {

using namespace ptx;

constexpr int BM = 128;
constexpr int EW_THREADS = 256;
constexpr int TMA_WARP = 8;
constexpr int MMA_WARP = 9;
constexpr int NTHREADS = 320;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_LIMIT = 232448;  // 227 KB per CTA
constexpr int SMEM_TAIL = 1024;     // barriers, TMEM base, abort flag, row-sum exchange
constexpr long long kTimeoutCycles = 2000000000LL;   // about a second
constexpr long long kPeerCheckCycles = 2000000LL;    // after ~1 ms also give up if another CTA timed out

template <int PASS, int D, int BN>
struct Cfg {
  static constexpr int NSTAT = PASS == 1 ? 2 : (PASS == 4 ? 4 : 3);
  static constexpr int NSTRM = PASS == 1 ? 2 : (PASS == 4 ? 3 : 4);
  static constexpr int NACC = PASS == 1 ? 2 : 4;
  static constexpr int NOUT = PASS >= 3 ? 2 : 0;
  static constexpr int OUT_COLS = NOUT * D;
  static constexpr int STAGE_COLS = NACC * BN;
  static constexpr int NSS = (TMEM_COLS - OUT_COLS) / STAGE_COLS >= 2 ? 2 : 1;  // score stages in TMEM
  static constexpr int STAT_BYTES = BM * D * 2;
  static constexpr int STRM_BYTES = BN * D * 2;
  static constexpr int SLOT_BYTES = NSTRM * STRM_BYTES;
  static constexpr int NSLOT_FIT = (SMEM_LIMIT - SMEM_TAIL - NSTAT * STAT_BYTES) / SLOT_BYTES;
  static constexpr int NSLOT = NSLOT_FIT > 4 ? 4 : NSLOT_FIT;
  static constexpr int SMEM_BYTES = NSTAT * STAT_BYTES + NSLOT * SLOT_BYTES + SMEM_TAIL;
  static constexpr int CH = BN / 32;  // 16-column chunks per elementwise thread (it owns BN/2 columns)
  static_assert(NSS * STAGE_COLS + OUT_COLS <= TMEM_COLS, "TMEM budget");
  static_assert(NSLOT >= 2, "need two streamed slots");
  static_assert(D == 64 || D == 128, "head dim");
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "streamed tile");
};

struct TcParams {
  CUtensorMap stat[4];
  CUtensorMap strm[4];
  const float* nlc;
  const float* nds;
  float* ndd;
  float* nbs;
  __nv_bfloat16* out0;
  __nv_bfloat16* out1;
  int* status;
  int n_q, n_k, causal, tiles_per_head;
  float scale;
};

struct Bars {
  uint64_t stat_full;
  uint64_t strm_full[4];
  uint64_t strm_free[4];
  uint64_t s_full[2];
  uint64_t s_free[2];
  uint64_t p_full;
  uint64_t out_full;
  uint64_t teardown;
  uint32_t tmem_base;
  int abort_flag;
  float red[BM];
};
static_assert(sizeof(Bars) <= SMEM_TAIL, "tail");

__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, Bars* b, int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  uint32_t spins = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0xFFu) == 0) {
      if (*reinterpret_cast<volatile int*>(&b->abort_flag)) return false;
      long long el = clock64() - start;
      if (el > kTimeoutCycles ||
          (el > kPeerCheckCycles && (*reinterpret_cast<volatile int*>(status) & FHOB_ERR_TIMEOUT))) {
        *reinterpret_cast<volatile int*>(&b->abort_flag) = 1;
        atomicOr(status, FHOB_ERR_TIMEOUT);
        return false;
      }
    }
  }
}

// D (+)= A . B^T with both tiles K-major in shared memory (rows of 64-element boxes, 128B swizzle).
template <int D, int A_ROWS, int B_ROWS>
__device__ __forceinline__ void gemm_ss(uint32_t d_tmem, uint32_t a_tile, uint32_t b_tile, uint32_t idesc,
                                        bool accumulate) {
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    uint32_t a = a_tile + (ks / 4) * (A_ROWS * 128) + (ks % 4) * 32;
    uint32_t b = b_tile + (ks / 4) * (B_ROWS * 128) + (ks % 4) * 32;
    umma_ss(d_tmem, umma_desc_sw128(a, 16, 1024), umma_desc_sw128(b, 16, 1024), idesc, (accumulate || ks > 0) ? 1u : 0u);
  }
}

// D (+)= A . B with A = bf16 tile in TMEM (128 x BN, 8 columns per 16 keys) and B = streamed
// tile (BN rows x D) read MN-major: the contraction runs down the BN rows.
template <int D, int BN>
__device__ __forceinline__ void gemm_ts(uint32_t d_tmem, uint32_t a_region, uint32_t b_tile, uint32_t idesc,
                                        bool accumulate) {
  constexpr int CH = BN / 32;
#pragma unroll
  for (int s = 0; s < BN / 16; ++s) {
    uint32_t a = a_region + (s / CH) * (BN / 2) + 8 * (s % CH);
    uint32_t b = b_tile + s * 2048;
    umma_ts(d_tmem, a, umma_desc_sw128(b, BN * 128, 1024), idesc, (accumulate || s > 0) ? 1u : 0u);
  }
}

template <int PASS, int D, int BN>
__global__ void __launch_bounds__(NTHREADS, 1) tc_pass_kernel(const __grid_constant__ TcParams p) {
  using C = Cfg<PASS, D, BN>;
  constexpr bool kQStat = PASS != 4;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* stat_tiles = smem;
  uint8_t* strm_tiles = smem + C::NSTAT * C::STAT_BYTES;
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

  int t_begin = 0, t_end = (n_strm + BN - 1) / BN;
  if (p.causal) {
    if (kQStat) {
      long last_key = static_cast<long>(m0) + BM - 1 + off;
      if (last_key < 0) t_end = 0;
      else if (last_key / BN + 1 < t_end) t_end = static_cast<int>(last_key / BN + 1);
    } else {
      long first_q = static_cast<long>(m0) - off;
      if (first_q > 0) t_begin = static_cast<int>(first_q / BN);
      if (t_begin > t_end) t_begin = t_end;
    }
  }
  const int n_iter = t_end - t_begin;

  // ---- set-up
  if (threadIdx.x == 0) {
    if (smem_u32(smem) & 1023u) atomicOr(p.status, FHOB_ERR_SMEM_ALIGN);
    mbar_init(&bars->stat_full, 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&bars->strm_full[i], 1);
      mbar_init(&bars->strm_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->s_free[i], EW_THREADS);
    }
    mbar_init(&bars->p_full, EW_THREADS);
    mbar_init(&bars->out_full, 1);
    mbar_init(&bars->teardown, 1);
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
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  if (warp == TMA_WARP) {
    // ================================================= TMA producer
    if (lane == 0 && n_iter > 0) {
      mbar_arrive_expect_tx(&bars->stat_full, C::NSTAT * C::STAT_BYTES);
      for (int i = 0; i < C::NSTAT; ++i)
        for (int bx = 0; bx < D / 64; ++bx)
          tma_load_3d(stat_tiles + i * C::STAT_BYTES + bx * (BM * 128), &p.stat[i], &bars->stat_full, bx * 64, m0,
                      head);
      int issued = 0;
      for (int it = 0; it < n_iter; ++it) {
        const int slot = it % C::NSLOT;
        if (!wait_bar(&bars->strm_free[slot], ((it / C::NSLOT) & 1) ^ 1, bars, p.status)) break;
        mbar_arrive_expect_tx(&bars->strm_full[slot], C::SLOT_BYTES);
        uint8_t* dst = strm_tiles + slot * C::SLOT_BYTES;
        const int n0 = (t_begin + it) * BN;
        for (int i = 0; i < C::NSTRM; ++i)
          for (int bx = 0; bx < D / 64; ++bx)
            tma_load_3d(dst + i * C::STRM_BYTES + bx * (BN * 128), &p.strm[i], &bars->strm_full[slot], bx * 64, n0,
                        head);
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
  } else if (warp == MMA_WARP) {
    // ================================================= MMA issuer
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BM, BN, false, false);
      constexpr uint32_t idesc_o = umma_idesc_bf16(BM, D, false, true);
      const uint32_t stat_base = smem_u32(stat_tiles);
      bool ok = wait_bar(&bars->stat_full, 0, bars, p.status);
      for (int it = 0; ok && it < n_iter; ++it) {
        const int slot = it % C::NSLOT;
        const int stage = it % C::NSS;
        ok = wait_bar(&bars->strm_full[slot], (it / C::NSLOT) & 1, bars, p.status);
        if (!ok) break;
        if (PASS <= 2) {
          ok = wait_bar(&bars->s_free[stage], ((it / C::NSS) & 1) ^ 1, bars, p.status);
          if (!ok) break;
        }
        tc_fence_after();
        const uint32_t strm_base = smem_u32(strm_tiles + slot * C::SLOT_BYTES);
        const uint32_t acc = tmem_base + C::OUT_COLS + stage * C::STAGE_COLS;
        auto st = [&](int i) { return stat_base + i * C::STAT_BYTES; };
        auto sr = [&](int i) { return strm_base + i * C::STRM_BYTES; };
        // score-shaped accumulators
        gemm_ss<D, BM, BN>(acc + 0 * BN, st(0), sr(0), idesc_s, false);  // S
        if (kQStat) {
          gemm_ss<D, BM, BN>(acc + 1 * BN, st(1), sr(0), idesc_s, false);  // ddQ K^T
          gemm_ss<D, BM, BN>(acc + 1 * BN, st(0), sr(1), idesc_s, true);   // + Q ddK^T
        } else {
          gemm_ss<D, BM, BN>(acc + 1 * BN, st(0), sr(1), idesc_s, false);  // K ddQ^T
          gemm_ss<D, BM, BN>(acc + 1 * BN, st(1), sr(0), idesc_s, true);   // + ddK Q^T
        }
        if (PASS >= 2) {
          gemm_ss<D, BM, BN>(acc + 2 * BN, st(2), sr(2), idesc_s, false);  // dP
          if (kQStat) gemm_ss<D, BM, BN>(acc + 3 * BN, st(2), sr(3), idesc_s, false);  // dO ddV^T
          else gemm_ss<D, BM, BN>(acc + 3 * BN, st(3), sr(2), idesc_s, false);         // ddV dO^T
        }
        umma_commit(&bars->s_full[stage]);
        if (PASS <= 2) {
          umma_commit(&bars->strm_free[slot]);
        } else {
          ok = wait_bar(&bars->p_full, it & 1, bars, p.status);
          if (!ok) break;
          tc_fence_after();
          const bool accum = it > 0;
          const uint32_t out0 = tmem_base, out1 = tmem_base + D;
          gemm_ts<D, BN>(out0, acc + 2 * BN, sr(1), idesc_o, accum);  // dS  . ddK | ddQ
          gemm_ts<D, BN>(out0, acc + 3 * BN, sr(0), idesc_o, true);   // dS2 . K   | Q
          gemm_ts<D, BN>(out1, acc + 1 * BN, sr(2), idesc_o, accum);  // ddP . V   | dO
          if (kQStat) gemm_ts<D, BN>(out1, acc + 0 * BN, sr(3), idesc_o, true);  // P . ddV
          umma_commit(&bars->strm_free[slot]);
        }
      }
      if (ok) {
        umma_commit(&bars->out_full);
      } else {
        // abort path: no tcgen05.mma may still be reading shared memory or TMEM at exit
        umma_commit(&bars->teardown);
        const long long start = clock64();
        while (!mbar_try_wait(&bars->teardown, 0)) {
          if (clock64() - start > kTimeoutCycles) break;
        }
      }
    }
  } else {
    // ================================================= elementwise warps
    const int quad = warp & 3, half = warp >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int g_row = m0 + row;  // stationary row of this thread
    const size_t vec_head = static_cast<size_t>(head) * p.n_q;
    const float scale = p.scale, sl2 = p.scale * kLog2e;

    float r_nlc = 0.f, r_nds = 0.f, r_ndd = 0.f, r_nbs = 0.f;
    if (kQStat && g_row < p.n_q) {
      r_nlc = p.nlc[vec_head + g_row];
      if (PASS >= 2) {
        r_nds = p.nds[vec_head + g_row];
        r_ndd = p.ndd[vec_head + g_row];
      }
      if (PASS >= 3) r_nbs = p.nbs[vec_head + g_row];
    }
    // visible streamed index range of this thread's row: lo <= idx <= hi
    int lo, hi;
    if (kQStat) {
      lo = 0;
      hi = p.n_k - 1;
      if (p.causal && g_row + off < hi) hi = g_row + off;
    } else {
      lo = p.causal ? g_row - off : 0;
      if (lo < 0) lo = 0;
      hi = p.n_q - 1;
    }
    float rowacc = 0.f;
    bool ok = true;

    for (int it = 0; it < n_iter; ++it) {
      const int stage = it % C::NSS;
      const int n0 = (t_begin + it) * BN;
      ok = __all_sync(0xffffffffu, wait_bar(&bars->s_full[stage], (it / C::NSS) & 1, bars, p.status));
      if (!ok) break;
      tc_fence_after();
      // does any element of this tile need masking?  (warp-uniform: depends on tile coordinates only)
      bool masked = n0 + BN > n_strm;
      if (p.causal) {
        if (kQStat) masked = masked || (n0 + BN - 1 > m0 + off);
        else masked = masked || (n0 + off < m0 + BM - 1);
      }
      const uint32_t acc = tmem_base + lane_base + C::OUT_COLS + stage * C::STAGE_COLS + half * (BN / 2);
#pragma unroll
      for (int c = 0; c < C::CH; ++c) {
        const int col0 = n0 + half * (BN / 2) + 16 * c;  // streamed index of this chunk's first column
        uint32_t s[16], a2[16], dp[16], x[16];
        tmem_ld16(acc + 0 * BN + 16 * c, s);
        tmem_ld16(acc + 1 * BN + 16 * c, a2);
        if (PASS >= 2) {
          tmem_ld16(acc + 2 * BN + 16 * c, dp);
          tmem_ld16(acc + 3 * BN + 16 * c, x);
        }
        tmem_wait_ld();
        uint32_t w_ds[8], w_ds2[8], w_ddp[8], w_p[8];
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
          float c_nlc[4], c_nds[4], c_ndd[4], c_nbs[4];
          if (kQStat) {
#pragma unroll
            for (int e = 0; e < 4; ++e) { c_nlc[e] = r_nlc; c_nds[e] = r_nds; c_ndd[e] = r_ndd; c_nbs[e] = r_nbs; }
          } else {
            const size_t vi = vec_head + col0 + 4 * j4;
            float4 v0 = __ldg(reinterpret_cast<const float4*>(p.nlc + vi));
            float4 v1 = __ldg(reinterpret_cast<const float4*>(p.nds + vi));
            float4 v2 = __ldg(reinterpret_cast<const float4*>(p.ndd + vi));
            float4 v3 = __ldg(reinterpret_cast<const float4*>(p.nbs + vi));
            c_nlc[0] = v0.x; c_nlc[1] = v0.y; c_nlc[2] = v0.z; c_nlc[3] = v0.w;
            c_nds[0] = v1.x; c_nds[1] = v1.y; c_nds[2] = v1.z; c_nds[3] = v1.w;
            c_ndd[0] = v2.x; c_ndd[1] = v2.y; c_ndd[2] = v2.z; c_ndd[3] = v2.w;
            c_nbs[0] = v3.x; c_nbs[1] = v3.y; c_nbs[2] = v3.z; c_nbs[3] = v3.w;
          }
          float o_ds[4], o_ds2[4], o_ddp[4], o_p[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = 4 * j4 + e;
            const float fs = __uint_as_float(s[j]), fa2 = __uint_as_float(a2[j]);
            bool allowed = true;
            if (masked) {
              const int idx = col0 + j;
              allowed = idx >= lo && idx <= hi;
            }
            float pr = ex2(fmaf(fs, sl2, c_nlc[e]));
            if (masked) pr = allowed ? pr : 0.f;
            if (PASS == 1) {
              rowacc = fmaf(pr, fa2, rowacc);
            } else {
              const float fdp = __uint_as_float(dp[j]), fx = __uint_as_float(x[j]);
              const float tt = fmaf(fa2, scale, c_ndd[e]);
              float u = fmaf(fdp, tt, fx);
              u = fmaf(c_nds[e], fa2, u);
              if (PASS == 2) {
                float term = pr * u;
                if (masked) term = allowed ? term : 0.f;
                rowacc += term;
              } else {
                o_ds[e] = pr * fmaf(fdp, scale, c_nds[e]);
                o_ds2[e] = pr * fmaf(u, scale, c_nbs[e]);
                o_ddp[e] = pr * tt;
                o_p[e] = pr;
                if (masked && !allowed) { o_ds[e] = 0.f; o_ds2[e] = 0.f; o_ddp[e] = 0.f; }
              }
            }
          }
          if (PASS >= 3) {
            w_ds[2 * j4] = pack_bf16(o_ds[0], o_ds[1]);
            w_ds[2 * j4 + 1] = pack_bf16(o_ds[2], o_ds[3]);
            w_ds2[2 * j4] = pack_bf16(o_ds2[0], o_ds2[1]);
            w_ds2[2 * j4 + 1] = pack_bf16(o_ds2[2], o_ds2[3]);
            w_ddp[2 * j4] = pack_bf16(o_ddp[0], o_ddp[1]);
            w_ddp[2 * j4 + 1] = pack_bf16(o_ddp[2], o_ddp[3]);
            if (PASS == 3) {
              w_p[2 * j4] = pack_bf16(o_p[0], o_p[1]);
              w_p[2 * j4 + 1] = pack_bf16(o_p[2], o_p[3]);
            }
          }
        }
        if (PASS >= 3) {
          // bf16 tiles overwrite the accumulator columns this thread has already consumed
          tmem_st8(acc + 2 * BN + 8 * c, w_ds);
          tmem_st8(acc + 3 * BN + 8 * c, w_ds2);
          tmem_st8(acc + 1 * BN + 8 * c, w_ddp);
          if (PASS == 3) tmem_st8(acc + 0 * BN + 8 * c, w_p);
        }
      }
      if (PASS <= 2) {
        tc_fence_before();
        mbar_arrive(&bars->s_free[stage]);
      } else {
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&bars->p_full);
      }
    }

    // ---- results
    if (PASS <= 2) {
      if (half == 1) bars->red[row] = rowacc;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (half == 0 && ok && g_row < p.n_q) {
        float tot = rowacc + bars->red[row];
        if (PASS == 1) p.ndd[vec_head + g_row] = -scale * tot;
        else p.nbs[vec_head + g_row] = -scale * tot;
      }
    } else {
      if (n_iter > 0) ok = ok && __all_sync(0xffffffffu, wait_bar(&bars->out_full, 0, bars, p.status));
      tc_fence_after();
      if (ok) {
#pragma unroll
        for (int o = 0; o < 2; ++o) {
          __nv_bfloat16* dst = (o == 0 ? p.out0 : p.out1) +
                               (static_cast<size_t>(head) * n_stat + (g_row < n_stat ? g_row : 0)) * D + half * (D / 2);
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t v[16];
            if (n_iter > 0) {
              tmem_ld16(tmem_base + lane_base + o * D + half * (D / 2) + 16 * c, v);
              tmem_wait_ld();
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = 0u;
            }
            if (g_row < n_stat) {
              uint4 w0, w1;
              w0.x = pack_bf16(__uint_as_float(v[0]), __uint_as_float(v[1]));
              w0.y = pack_bf16(__uint_as_float(v[2]), __uint_as_float(v[3]));
              w0.z = pack_bf16(__uint_as_float(v[4]), __uint_as_float(v[5]));
              w0.w = pack_bf16(__uint_as_float(v[6]), __uint_as_float(v[7]));
              w1.x = pack_bf16(__uint_as_float(v[8]), __uint_as_float(v[9]));
              w1.y = pack_bf16(__uint_as_float(v[10]), __uint_as_float(v[11]));
              w1.z = pack_bf16(__uint_as_float(v[12]), __uint_as_float(v[13]));
              w1.w = pack_bf16(__uint_as_float(v[14]), __uint_as_float(v[15]));
              uint4* d4 = reinterpret_cast<uint4*>(dst + 16 * c);
              d4[0] = w0;
              d4[1] = w1;
            }
          }
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
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// (bh, n, d) bf16 row-major tensor, box = 64 columns x `rows` rows of one head, 128-byte swizzle.
int make_map(CUtensorMap* m, const void* base, int bh, int n, int d, int rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_cuda_error_text("cuTensorMapEncodeTiled entry point not available");
    return FHOB_ERR_CUDA;
  }
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(bh)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(d) * 2, static_cast<cuuint64_t>(n) * d * 2};
  cuuint32_t box[3] = {64, static_cast<cuuint32_t>(rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[96];
    snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    set_cuda_error_text(buf);
    return FHOB_ERR_CUDA;
  }
  return FHOB_OK;
}

template <int PASS, int D, int BN>
int launch(const FhobProblem& p, cudaStream_t s) {
  using C = Cfg<PASS, D, BN>;
  RowVectors rv = row_vectors(p);
  TcParams tp;
  memset(&tp, 0, sizeof(tp));
  const void* q_side[3] = {p.q, p.ddq, p.d_o};
  const void* k_side[4] = {p.k, p.ddk, p.v, p.ddv};
  int st = FHOB_OK;
  if (PASS != 4) {
    for (int i = 0; i < C::NSTAT && st == FHOB_OK; ++i) st = make_map(&tp.stat[i], q_side[i], p.bh, p.n_q, D, BM);
    for (int i = 0; i < C::NSTRM && st == FHOB_OK; ++i) st = make_map(&tp.strm[i], k_side[i], p.bh, p.n_k, D, BN);
  } else {
    for (int i = 0; i < C::NSTAT && st == FHOB_OK; ++i) st = make_map(&tp.stat[i], k_side[i], p.bh, p.n_k, D, BM);
    for (int i = 0; i < C::NSTRM && st == FHOB_OK; ++i) st = make_map(&tp.strm[i], q_side[i], p.bh, p.n_q, D, BN);
  }
  if (st != FHOB_OK) return st;
  tp.nlc = rv.nlc; tp.nds = rv.nds; tp.ndd = rv.ndd; tp.nbs = rv.nbs;
  tp.out0 = static_cast<__nv_bfloat16*>(PASS == 3 ? p.dq2 : p.dk2);
  tp.out1 = static_cast<__nv_bfloat16*>(PASS == 3 ? p.ddo : p.dv2);
  tp.status = rv.status;
  tp.n_q = p.n_q; tp.n_k = p.n_k; tp.causal = p.causal; tp.scale = p.scale;
  const int n_stat = PASS == 4 ? p.n_k : p.n_q;
  tp.tiles_per_head = (n_stat + BM - 1) / BM;
  FHOB_CUDA_OK(cudaFuncSetAttribute(tc_pass_kernel<PASS, D, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    C::SMEM_BYTES));
  const long long blocks = static_cast<long long>(tp.tiles_per_head) * p.bh;
  if (blocks > 0x7fffffffLL) return FHOB_ERR_SHAPE;
  tc_pass_kernel<PASS, D, BN><<<static_cast<unsigned>(blocks), NTHREADS, C::SMEM_BYTES, s>>>(tp);
  FHOB_CUDA_OK(cudaGetLastError());
  return FHOB_OK;
}

template <int D>
int dispatch(int pass, const FhobProblem& p, cudaStream_t s) {
  switch (pass) {
    case 1: return launch<1, D, 64>(p, s);
    case 2: return launch<2, D, 64>(p, s);
    case 3: return launch<3, D, 64>(p, s);
    case 4: return launch<4, D, 64>(p, s);
  }
  return FHOB_ERR_ARG;
}

}  // namespace

bool tc_supported(const FhobProblem& p) {
  return p.dtype == FHOB_BF16 && (p.d == 64 || p.d == 128) && (p.n_q % 4 == 0);
}

int tc_pass(int pass, const FhobProblem& p, cudaStream_t s) {
  if (!tc_supported(p)) return FHOB_ERR_SHAPE;
  static thread_local int checked_dev = -1;
  int dev = 0;
  FHOB_CUDA_OK(cudaGetDevice(&dev));
  if (dev != checked_dev) {
    int major = 0;
    FHOB_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) return FHOB_ERR_ARCH;
    checked_dev = dev;
  }
  return p.d == 64 ? dispatch<64>(pass, p, s) : dispatch<128>(pass, p, s);
}

}  // namespace fhob
