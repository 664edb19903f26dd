// CUDA-core (FFMA) kernels of the double-backward attention operator.
//
// They serve fp32 problems, where bf16 tensor-core products could not reach a
// 1e-4 relative error, and any bf16 problem the caller forces onto them.  The
// algorithm is the same four recomputation passes as the tensor-core kernels
// (reference: fhog/triton_bwdbwd.py:178-313 for the query-tiled passes 1-3,
// :321-535 for the key-tiled pass 4): a CTA keeps TM "stationary" rows in
// shared memory, streams TN rows of the other side per step, rebuilds the four
// score-shaped tiles S, A2, dP, X from fp32 dot products, applies the
// elementwise formulas of fhob_common.cuh and either reduces along the row
// (passes 1, 2) or feeds the resulting tiles into the output products
// (passes 3, 4).  Arbitrary n_q, n_k and head dims <= 128 are handled by bounds
// checks; pairs outside the matrix or hidden by the causal mask contribute zero.
// Two head dims: Q, K, ddQ, ddK, dQ2, dK2 have `d` columns, V, ddV, dO, O, ddO, dV2
// have `dv` (jax_refs/flash_impl.py:381-389 has d_in != d_out); shared-memory
// tiles all use the row pitch of the larger one.
#include "fhob_common.cuh"

namespace fhob {
namespace {

constexpr int TM = 32;        // stationary rows per CTA
constexpr int TN = 32;        // streamed rows per step
constexpr int NT = 256;       // threads per CTA: 8 warps, warp w owns rows 4w..4w+3, lane = column
constexpr int RPW = TM / 8;   // rows per warp
constexpr int DCH = 4;        // output columns per thread and row: lane + 32*m, m < DCH  (d <= 128)

struct SimtParams {
  const void *q, *k, *v, *d_o, *ddq, *ddk, *ddv;
  void *dq2, *dk2, *dv2, *ddo;
  const float *nlc, *k1;
  float *ndd, *k23;
  int bh, n_q, n_k, d, dv, causal, window;
  float scale;
};

// Grid of (stationary tiles, heads): heads beyond what grid.y can index continue in grid.z.
constexpr int kMaxGridY = 65535;
inline dim3 head_grid(int tiles, int bh) {
  return dim3(tiles, bh < kMaxGridY ? bh : kMaxGridY, (bh + kMaxGridY - 1) / kMaxGridY);
}

template <typename T>
__device__ __forceinline__ float ld_elem(const void* p, size_t i);
template <>
__device__ __forceinline__ float ld_elem<float>(const void* p, size_t i) {
  return static_cast<const float*>(p)[i];
}
template <>
__device__ __forceinline__ float ld_elem<__nv_bfloat16>(const void* p, size_t i) {
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
template <>
__device__ __forceinline__ float ld_elem<__half>(const void* p, size_t i) {
  return __half2float(static_cast<const __half*>(p)[i]);
}
template <typename T>
__device__ __forceinline__ void st_elem(void* p, size_t i, float v);
template <>
__device__ __forceinline__ void st_elem<__half>(void* p, size_t i, float v) {
  static_cast<__half*>(p)[i] = __float2half_rn(v);
}
template <>
__device__ __forceinline__ void st_elem<float>(void* p, size_t i, float v) {
  static_cast<float*>(p)[i] = v;
}
template <>
__device__ __forceinline__ void st_elem<__nv_bfloat16>(void* p, size_t i, float v) {
  static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// Loads rows [row0, row0+rows) of a (n, d) matrix into a [rows][ld] fp32 tile, zero beyond n.
template <typename T>
__device__ __forceinline__ void load_tile(float* tile, int ld, const void* src, size_t head_off,
                                          int row0, int rows, int n, int d) {
  for (int idx = threadIdx.x; idx < rows * d; idx += NT) {
    int r = idx / d, c = idx - r * d;
    int gr = row0 + r;
    tile[r * ld + c] = gr < n ? ld_elem<T>(src, head_off + static_cast<size_t>(gr) * d + c) : 0.f;
  }
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}

// PASS 1..3: stationary = query tile, streamed = key tiles.
// PASS 4:    stationary = key tile,   streamed = query tiles.
template <typename T, int PASS>
__global__ void __launch_bounds__(NT) simt_pass_kernel(const SimtParams p) {
  extern __shared__ float smem[];
  const int d = p.d, dv = p.dv;
  const int ld = (d > dv ? d : dv) + 1;
  constexpr bool kQStationary = PASS != 4;
  float* stat[4];
  float* strm[4];
  for (int i = 0; i < 4; ++i) stat[i] = smem + i * TM * ld;
  for (int i = 0; i < 4; ++i) strm[i] = smem + (4 * TM + i * TN) * ld;
  float* sacc = smem + (4 * TM + 4 * TN) * ld;     // [4][TM][TN+1]: S, A2, dP, X
  float* ptile = sacc + 4 * TM * (TN + 1);          // [4][TM][TN+1]: P-type tiles
  float* svec = ptile + 4 * TM * (TN + 1);          // [4][TN]: row vectors of streamed queries (pass 4)
  constexpr int LT = TN + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * TM;
  const int bh = blockIdx.y + blockIdx.z * kMaxGridY;   // see head_grid
  if (bh >= p.bh) return;
  const size_t qoff = static_cast<size_t>(bh) * p.n_q * d, qoff_v = static_cast<size_t>(bh) * p.n_q * dv;
  const size_t koff = static_cast<size_t>(bh) * p.n_k * d, koff_v = static_cast<size_t>(bh) * p.n_k * dv;
  const size_t voff = static_cast<size_t>(bh) * row_stride(p.n_q);  // row-vector offset
  const int causal_off = p.n_k - p.n_q;
  const int n_stat = kQStationary ? p.n_q : p.n_k;
  const int n_strm = kQStationary ? p.n_k : p.n_q;

  if (kQStationary) {
    load_tile<T>(stat[0], ld, p.q, qoff, m0, TM, p.n_q, d);
    load_tile<T>(stat[1], ld, p.ddq, qoff, m0, TM, p.n_q, d);
    if (PASS >= 2) load_tile<T>(stat[2], ld, p.d_o, qoff_v, m0, TM, p.n_q, dv);
  } else {
    load_tile<T>(stat[0], ld, p.k, koff, m0, TM, p.n_k, d);
    load_tile<T>(stat[1], ld, p.ddk, koff, m0, TM, p.n_k, d);
    load_tile<T>(stat[2], ld, p.v, koff_v, m0, TM, p.n_k, dv);
    load_tile<T>(stat[3], ld, p.ddv, koff_v, m0, TM, p.n_k, dv);
  }

  // per-row constants of the stationary queries (passes 1-3)
  float r_nlc[RPW], r_k1[RPW], r_nds[RPW], r_ndd[RPW], r_nbs[RPW], rowacc[RPW];
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    int qi = m0 + warp * RPW + i;
    bool ok = kQStationary && qi < p.n_q;
    r_nlc[i] = ok ? p.nlc[voff + qi] : 0.f;
    const float k1 = ok && PASS >= 2 ? p.k1[voff + qi] : 0.f;
    r_k1[i] = k1;
    r_nds[i] = k1 * p.scale;                                                    // -D*scale
    r_ndd[i] = ok && PASS >= 2 ? p.ndd[voff + qi] : 0.f;
    r_nbs[i] = ok && PASS >= 3 ? (p.k23[voff + qi] + k1 * r_ndd[i]) * p.scale : 0.f;  // -b*scale
    rowacc[i] = 0.f;
  }
  float out0[RPW][DCH], out1[RPW][DCH];
#pragma unroll
  for (int i = 0; i < RPW; ++i)
#pragma unroll
    for (int m = 0; m < DCH; ++m) out0[i][m] = out1[i][m] = 0.f;

  // streamed range
  int t_begin, t_end;
  visible_tiles(kQStationary, m0, TM, TN, n_strm, causal_off, p.causal, p.window, t_begin, t_end);
  const float sl2 = p.scale * kLog2e;

  for (int t = t_begin; t < t_end; ++t) {
    const int n0 = t * TN;
    __syncthreads();  // previous step finished with strm/ptile
    if (kQStationary) {
      load_tile<T>(strm[0], ld, p.k, koff, n0, TN, p.n_k, d);
      load_tile<T>(strm[1], ld, p.ddk, koff, n0, TN, p.n_k, d);
      if (PASS >= 2) {
        load_tile<T>(strm[2], ld, p.v, koff_v, n0, TN, p.n_k, dv);
        load_tile<T>(strm[3], ld, p.ddv, koff_v, n0, TN, p.n_k, dv);
      }
    } else {
      load_tile<T>(strm[0], ld, p.q, qoff, n0, TN, p.n_q, d);
      load_tile<T>(strm[1], ld, p.ddq, qoff, n0, TN, p.n_q, d);
      load_tile<T>(strm[2], ld, p.d_o, qoff_v, n0, TN, p.n_q, dv);
      if (threadIdx.x < TN) {
        int qi = n0 + threadIdx.x;
        bool ok = qi < p.n_q;
        svec[0 * TN + threadIdx.x] = ok ? p.nlc[voff + qi] : 0.f;
        const float k1 = ok ? p.k1[voff + qi] : 0.f, ndd = ok ? p.ndd[voff + qi] : 0.f;
        svec[1 * TN + threadIdx.x] = k1 * p.scale;
        svec[2 * TN + threadIdx.x] = ndd;
        svec[3 * TN + threadIdx.x] = ok ? (p.k23[voff + qi] + k1 * ndd) * p.scale : 0.f;
      }
    }
    __syncthreads();

    // score-shaped tiles: rows = stationary, columns = streamed; this thread: RPW rows x column `lane`
    float s[RPW], a2[RPW], dp[RPW], x[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) s[i] = a2[i] = dp[i] = x[i] = 0.f;
    for (int e = 0; e < d; ++e) {   // contractions over the q/k head dim
      float c0 = strm[0][lane * ld + e], c1 = strm[1][lane * ld + e];
#pragma unroll
      for (int i = 0; i < RPW; ++i) {
        int r = warp * RPW + i;
        float a0 = stat[0][r * ld + e], a1 = stat[1][r * ld + e];
        s[i] = fmaf(a0, c0, s[i]);
        a2[i] = fmaf(a1, c0, fmaf(a0, c1, a2[i]));
      }
    }
    if (PASS >= 2) {
      for (int e = 0; e < dv; ++e) {   // contractions over the v head dim
        float c2 = strm[2][lane * ld + e];
        float c3 = kQStationary ? strm[3][lane * ld + e] : 0.f;
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
          int r = warp * RPW + i;
          float a2v = stat[2][r * ld + e];
          dp[i] = fmaf(a2v, c2, dp[i]);
          if (kQStationary) x[i] = fmaf(a2v, c3, x[i]);
          else x[i] = fmaf(stat[3][r * ld + e], c2, x[i]);
        }
      }
    }

    // elementwise
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      int r = warp * RPW + i;
      int qi = kQStationary ? m0 + r : n0 + lane;
      int kj = kQStationary ? n0 + lane : m0 + r;
      bool allowed = qi < p.n_q && kj < p.n_k && pair_visible(qi, kj, causal_off, p.causal, p.window);
      float nlc, nds, ndd, nbs;
      if (kQStationary) { nlc = r_nlc[i]; nds = r_nds[i]; ndd = r_ndd[i]; nbs = r_nbs[i]; }
      else { nlc = svec[lane]; nds = svec[TN + lane]; ndd = svec[2 * TN + lane]; nbs = svec[3 * TN + lane]; }
      float pr = allowed ? exp2f(fmaf(s[i], sl2, nlc)) : 0.f;
      if (PASS == 1) {
        rowacc[i] = fmaf(pr, a2[i], rowacc[i]);
      } else {
        float tt = fmaf(a2[i], p.scale, ndd);
        float u = fmaf(dp[i], tt, x[i]);
        u = fmaf(nds, a2[i], u);
        if (PASS == 2) {
          rowacc[i] = fmaf(pr, u, rowacc[i]);
        } else {
          ptile[(0 * TM + r) * LT + lane] = pr * fmaf(dp[i], p.scale, nds);  // dS
          ptile[(1 * TM + r) * LT + lane] = pr * fmaf(u, p.scale, nbs);      // dS2
          ptile[(2 * TM + r) * LT + lane] = pr * tt;                          // ddP
          ptile[(3 * TM + r) * LT + lane] = pr;                               // P
        }
      }
    }

    if (PASS >= 3) {
      __syncwarp();  // a warp only reads the ptile rows it wrote itself
      // PASS 3: out0 = dQ2 += dS ddK + dS2 K ;  out1 = ddO += ddP V + P ddV
      // PASS 4: out0 = dK2 += dS ddQ + dS2 Q ;  out1 = dV2 += ddP dO
      const float* b_ds = kQStationary ? strm[1] : strm[1];   // ddK | ddQ
      const float* b_ds2 = kQStationary ? strm[0] : strm[0];  // K   | Q
      const float* b_ddp = kQStationary ? strm[2] : strm[2];  // V   | dO
      for (int c = 0; c < TN; ++c) {
        float bds[DCH], bds2[DCH], bddp[DCH], bp[DCH];
#pragma unroll
        for (int m = 0; m < DCH; ++m) {
          int col = lane + 32 * m;
          bool in = col < d, in_v = col < dv;
          bds[m] = in ? b_ds[c * ld + col] : 0.f;
          bds2[m] = in ? b_ds2[c * ld + col] : 0.f;
          bddp[m] = in_v ? b_ddp[c * ld + col] : 0.f;
          bp[m] = (in_v && kQStationary) ? strm[3][c * ld + col] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
          int r = warp * RPW + i;
          float vds = ptile[(0 * TM + r) * LT + c], vds2 = ptile[(1 * TM + r) * LT + c];
          float vddp = ptile[(2 * TM + r) * LT + c], vp = ptile[(3 * TM + r) * LT + c];
#pragma unroll
          for (int m = 0; m < DCH; ++m) {
            out0[i][m] = fmaf(vds, bds[m], fmaf(vds2, bds2[m], out0[i][m]));
            out1[i][m] = fmaf(vddp, bddp[m], out1[i][m]);
            if (kQStationary) out1[i][m] = fmaf(vp, bp[m], out1[i][m]);
          }
        }
      }
    }
  }

  // results
  if (PASS <= 2) {
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      float tot = warp_sum(rowacc[i]);
      int qi = m0 + warp * RPW + i;
      if (lane == 0 && qi < p.n_q) {
        if (PASS == 1) p.ndd[voff + qi] = -p.scale * tot;          // -dd, dd = scale * sum P A2
        else p.k23[voff + qi] = -r_k1[i] * r_ndd[i] - tot;          // -D*dd - b, b = sum P dP2
      }
    }
  } else {
    void* o0 = kQStationary ? p.dq2 : p.dk2;
    void* o1 = kQStationary ? p.ddo : p.dv2;
    size_t off = kQStationary ? qoff : koff, off_v = kQStationary ? qoff_v : koff_v;
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      int gr = m0 + warp * RPW + i;
      if (gr >= n_stat) continue;
#pragma unroll
      for (int m = 0; m < DCH; ++m) {
        int col = lane + 32 * m;
        if (col < d) st_elem<T>(o0, off + static_cast<size_t>(gr) * d + col, out0[i][m]);
        if (col < dv) st_elem<T>(o1, off_v + static_cast<size_t>(gr) * dv + col, out1[i][m]);
      }
    }
  }
}

// O(N)-memory forward: online softmax over key tiles.
template <typename T>
__global__ void __launch_bounds__(NT) simt_forward_kernel(const SimtParams p, void* o_out, float* lse_out) {
  extern __shared__ float smem[];
  const int d = p.d, dv = p.dv, ld = (d > dv ? d : dv) + 1;
  float* qs = smem;
  float* ks = qs + TM * ld;
  float* vs = ks + TN * ld;
  float* ps = vs + TN * ld;  // [TM][TN+1]
  constexpr int LT = TN + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * TM, bh = blockIdx.y + blockIdx.z * kMaxGridY;   // see head_grid
  if (bh >= p.bh) return;
  const size_t qoff = static_cast<size_t>(bh) * p.n_q * d, qoff_v = static_cast<size_t>(bh) * p.n_q * dv;
  const size_t koff = static_cast<size_t>(bh) * p.n_k * d, koff_v = static_cast<size_t>(bh) * p.n_k * dv;
  const int causal_off = p.n_k - p.n_q;
  load_tile<T>(qs, ld, p.q, qoff, m0, TM, p.n_q, d);
  float mrow[RPW], lrow[RPW], acc[RPW][DCH];
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    mrow[i] = -INFINITY;
    lrow[i] = 0.f;
#pragma unroll
    for (int m = 0; m < DCH; ++m) acc[i][m] = 0.f;
  }
  int t_begin, t_end;
  visible_tiles(true, m0, TM, TN, p.n_k, causal_off, p.causal, p.window, t_begin, t_end);
  const float sl2 = p.scale * kLog2e;
  for (int t = t_begin; t < t_end; ++t) {
    const int n0 = t * TN;
    __syncthreads();
    load_tile<T>(ks, ld, p.k, koff, n0, TN, p.n_k, d);
    if (o_out) load_tile<T>(vs, ld, p.v, koff_v, n0, TN, p.n_k, dv);
    __syncthreads();
    float s[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) s[i] = 0.f;
    for (int e = 0; e < d; ++e) {
      float c0 = ks[lane * ld + e];
#pragma unroll
      for (int i = 0; i < RPW; ++i) s[i] = fmaf(qs[(warp * RPW + i) * ld + e], c0, s[i]);
    }
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      int r = warp * RPW + i, qi = m0 + r, kj = n0 + lane;
      bool allowed = qi < p.n_q && kj < p.n_k && pair_visible(qi, kj, causal_off, p.causal, p.window);
      float sv = allowed ? s[i] * sl2 : -INFINITY;  // log2 domain
      float mnew = fmaxf(mrow[i], warp_max(sv));
      float alpha = (mnew == -INFINITY) ? 1.f : exp2f(mrow[i] - mnew);
      float pv = (mnew == -INFINITY) ? 0.f : exp2f(sv - mnew);
      lrow[i] = lrow[i] * alpha + warp_sum(pv);
      mrow[i] = mnew;
      ps[r * LT + lane] = pv;
#pragma unroll
      for (int m = 0; m < DCH; ++m) acc[i][m] *= alpha;
    }
    __syncwarp();
    for (int c = 0; c < TN; ++c) {
      float bv[DCH];
#pragma unroll
      for (int m = 0; m < DCH; ++m) {
        int col = lane + 32 * m;
        bv[m] = (col < dv && o_out) ? vs[c * ld + col] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < RPW; ++i) {
        float pv = ps[(warp * RPW + i) * LT + c];
#pragma unroll
        for (int m = 0; m < DCH; ++m) acc[i][m] = fmaf(pv, bv[m], acc[i][m]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    int qi = m0 + warp * RPW + i;
    if (qi >= p.n_q) continue;
    float inv = lrow[i] > 0.f ? 1.f / lrow[i] : 0.f;
#pragma unroll
    for (int m = 0; m < DCH; ++m) {
      int col = lane + 32 * m;
      if (col < dv && o_out) st_elem<T>(o_out, qoff_v + static_cast<size_t>(qi) * dv + col, acc[i][m] * inv);
    }
    if (lane == 0)
      lse_out[static_cast<size_t>(bh) * p.n_q + qi] =
          lrow[i] > 0.f ? (mrow[i] + log2f(lrow[i])) * 0.6931471805599453f : -INFINITY;
  }
}

// First backward (dQ | dK, dV) of attention from the saved forward results, O(N) memory.
// KSIDE = false: a CTA owns TM queries and streams keys:   dQ = scale * (P (dP - D)) K.
// KSIDE = true:  a CTA owns TM keys and streams queries:   dV = P^T dO,  dK = scale * (P (dP - D))^T Q.
// Reads nlc = -L*log2(e) and k1 = -D from the workspace (written by the pre-pass).
template <typename T, bool KSIDE>
__global__ void __launch_bounds__(NT) simt_backward_kernel(const SimtParams p, void* out0, void* out1) {
  extern __shared__ float smem[];
  const int d = p.d, dv = p.dv, ld = (d > dv ? d : dv) + 1;
  float* stat0 = smem;                       // Q | K
  float* stat1 = stat0 + TM * ld;            // dO | V
  float* strm0 = stat1 + TM * ld;            // K | Q
  float* strm1 = strm0 + TN * ld;            // V | dO
  float* pt = strm1 + TN * ld;               // [2][TM][TN+1]: P and dS tiles
  float* svec = pt + 2 * TM * (TN + 1);      // [2][TN]: nlc, k1 of streamed queries (KSIDE)
  constexpr int LT = TN + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * TM, bh = blockIdx.y + blockIdx.z * kMaxGridY;   // see head_grid
  if (bh >= p.bh) return;
  const size_t qoff = static_cast<size_t>(bh) * p.n_q * d, qoff_v = static_cast<size_t>(bh) * p.n_q * dv;
  const size_t koff = static_cast<size_t>(bh) * p.n_k * d, koff_v = static_cast<size_t>(bh) * p.n_k * dv;
  const size_t voff = static_cast<size_t>(bh) * row_stride(p.n_q);
  const int causal_off = p.n_k - p.n_q;
  const int n_stat = KSIDE ? p.n_k : p.n_q, n_strm = KSIDE ? p.n_q : p.n_k;
  if (KSIDE) {
    load_tile<T>(stat0, ld, p.k, koff, m0, TM, p.n_k, d);
    load_tile<T>(stat1, ld, p.v, koff_v, m0, TM, p.n_k, dv);
  } else {
    load_tile<T>(stat0, ld, p.q, qoff, m0, TM, p.n_q, d);
    load_tile<T>(stat1, ld, p.d_o, qoff_v, m0, TM, p.n_q, dv);
  }
  float r_nlc[RPW], r_k1[RPW];
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    const int qi = m0 + warp * RPW + i;
    const bool ok = !KSIDE && qi < p.n_q;
    r_nlc[i] = ok ? p.nlc[voff + qi] : 0.f;
    r_k1[i] = ok ? p.k1[voff + qi] : 0.f;
  }
  float acc0[RPW][DCH], acc1[RPW][DCH];
#pragma unroll
  for (int i = 0; i < RPW; ++i)
#pragma unroll
    for (int m = 0; m < DCH; ++m) acc0[i][m] = acc1[i][m] = 0.f;
  int t_begin, t_end;
  visible_tiles(!KSIDE, m0, TM, TN, n_strm, causal_off, p.causal, p.window, t_begin, t_end);
  const float sl2 = p.scale * kLog2e;
  for (int t = t_begin; t < t_end; ++t) {
    const int n0 = t * TN;
    __syncthreads();
    if (KSIDE) {
      load_tile<T>(strm0, ld, p.q, qoff, n0, TN, p.n_q, d);
      load_tile<T>(strm1, ld, p.d_o, qoff_v, n0, TN, p.n_q, dv);
      if (threadIdx.x < TN) {
        const int qi = n0 + threadIdx.x;
        svec[threadIdx.x] = qi < p.n_q ? p.nlc[voff + qi] : 0.f;
        svec[TN + threadIdx.x] = qi < p.n_q ? p.k1[voff + qi] : 0.f;
      }
    } else {
      load_tile<T>(strm0, ld, p.k, koff, n0, TN, p.n_k, d);
      load_tile<T>(strm1, ld, p.v, koff_v, n0, TN, p.n_k, dv);
    }
    __syncthreads();
    float s[RPW], dp[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) s[i] = dp[i] = 0.f;
    for (int e = 0; e < d; ++e) {
      const float c0 = strm0[lane * ld + e];
#pragma unroll
      for (int i = 0; i < RPW; ++i) s[i] = fmaf(stat0[(warp * RPW + i) * ld + e], c0, s[i]);
    }
    for (int e = 0; e < dv; ++e) {
      const float c1 = strm1[lane * ld + e];
#pragma unroll
      for (int i = 0; i < RPW; ++i) dp[i] = fmaf(stat1[(warp * RPW + i) * ld + e], c1, dp[i]);
    }
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      const int r = warp * RPW + i;
      const int qi = KSIDE ? n0 + lane : m0 + r, kj = KSIDE ? m0 + r : n0 + lane;
      const bool allowed = qi < p.n_q && kj < p.n_k && pair_visible(qi, kj, causal_off, p.causal, p.window);
      const float nlc = KSIDE ? svec[lane] : r_nlc[i], k1 = KSIDE ? svec[TN + lane] : r_k1[i];
      const float pr = allowed ? exp2f(fmaf(s[i], sl2, nlc)) : 0.f;
      pt[(0 * TM + r) * LT + lane] = pr;
      pt[(1 * TM + r) * LT + lane] = allowed ? pr * (dp[i] + k1) * p.scale : 0.f;  // dS
    }
    __syncwarp();
    for (int c = 0; c < TN; ++c) {
      float b0[DCH], b1[DCH];
#pragma unroll
      for (int m = 0; m < DCH; ++m) {
        const int col = lane + 32 * m;
        b0[m] = col < d ? strm0[c * ld + col] : 0.f;    // K | Q
        b1[m] = col < dv ? strm1[c * ld + col] : 0.f;   // V | dO
      }
#pragma unroll
      for (int i = 0; i < RPW; ++i) {
        const int r = warp * RPW + i;
        const float vp = pt[(0 * TM + r) * LT + c], vds = pt[(1 * TM + r) * LT + c];
#pragma unroll
        for (int m = 0; m < DCH; ++m) {
          acc0[i][m] = fmaf(vds, b0[m], acc0[i][m]);              // dQ += dS K   | dK += dS^T Q
          if (KSIDE) acc1[i][m] = fmaf(vp, b1[m], acc1[i][m]);    //              | dV += P^T dO
        }
      }
    }
  }
  const size_t off = KSIDE ? koff : qoff;
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    const int gr = m0 + warp * RPW + i;
    if (gr >= n_stat) continue;
#pragma unroll
    for (int m = 0; m < DCH; ++m) {
      const int col = lane + 32 * m;
      if (col < d) st_elem<T>(out0, off + static_cast<size_t>(gr) * d + col, acc0[i][m]);
      if (KSIDE && col < dv) st_elem<T>(out1, koff_v + static_cast<size_t>(gr) * dv + col, acc1[i][m]);
    }
  }
}


int pitch(const FhobProblem& p) {  // row pitch of the shared-memory tiles: the larger head dim + 1
  const int dv = head_dim_v(p);
  return (p.d > dv ? p.d : dv) + 1;
}

size_t pass_smem_bytes(const FhobProblem& p) {
  size_t ld = pitch(p);
  return sizeof(float) * ((4 * TM + 4 * TN) * ld + 8 * TM * (TN + 1) + 4 * TN);
}

SimtParams make_params(const FhobProblem& p) {
  RowVectors rv = row_vectors(p);
  SimtParams s;
  s.q = p.q; s.k = p.k; s.v = p.v; s.d_o = p.d_o; s.ddq = p.ddq; s.ddk = p.ddk; s.ddv = p.ddv;
  s.dq2 = p.dq2; s.dk2 = p.dk2; s.dv2 = p.dv2; s.ddo = p.ddo;
  s.nlc = rv.nlc; s.k1 = rv.k1; s.ndd = rv.ndd; s.k23 = rv.k23;
  s.bh = p.bh; s.n_q = p.n_q; s.n_k = p.n_k; s.d = p.d; s.dv = head_dim_v(p); s.causal = p.causal; s.window = p.window; s.scale = p.scale;
  return s;
}

template <typename T, int PASS>
int launch_pass(const FhobProblem& p, cudaStream_t st) {
  size_t smem = pass_smem_bytes(p);
  FHOB_CUDA_OK(cudaFuncSetAttribute(simt_pass_kernel<T, PASS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(smem)));
  int n_stat = PASS == 4 ? p.n_k : p.n_q;
  dim3 grid = head_grid((n_stat + TM - 1) / TM, p.bh);
  simt_pass_kernel<T, PASS><<<grid, NT, smem, st>>>(make_params(p));
  FHOB_CUDA_OK(cudaGetLastError());
  return FHOB_OK;
}

template <typename T>
int dispatch_pass(int pass, const FhobProblem& p, cudaStream_t st) {
  switch (pass) {
    case 1: return launch_pass<T, 1>(p, st);
    case 2: return launch_pass<T, 2>(p, st);
    case 3: return launch_pass<T, 3>(p, st);
    case 4: return launch_pass<T, 4>(p, st);
  }
  return FHOB_ERR_ARG;
}

template <typename T>
int launch_backward(const FhobProblem& p, void* dq, void* dk, void* dv, cudaStream_t st) {
  const size_t smem = sizeof(float) * ((2 * TM + 2 * TN) * pitch(p) + 2 * TM * (TN + 1) + 2 * TN);
  SimtParams s = make_params(p);
  FHOB_CUDA_OK(cudaFuncSetAttribute(simt_backward_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(smem)));
  FHOB_CUDA_OK(cudaFuncSetAttribute(simt_backward_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(smem)));
  simt_backward_kernel<T, false><<<head_grid((p.n_q + TM - 1) / TM, p.bh), NT, smem, st>>>(s, dq, nullptr);
  FHOB_CUDA_OK(cudaGetLastError());
  simt_backward_kernel<T, true><<<head_grid((p.n_k + TM - 1) / TM, p.bh), NT, smem, st>>>(s, dk, dv);
  FHOB_CUDA_OK(cudaGetLastError());
  return FHOB_OK;
}

}  // namespace

int simt_backward(const FhobProblem& p, void* dq, void* dk, void* dv, cudaStream_t st) {
  if (p.d > 32 * DCH || head_dim_v(p) > 32 * DCH) return FHOB_ERR_SHAPE;
  if (p.dtype == FHOB_F32) return launch_backward<float>(p, dq, dk, dv, st);
  if (p.dtype == FHOB_F16) return launch_backward<__half>(p, dq, dk, dv, st);
  return launch_backward<__nv_bfloat16>(p, dq, dk, dv, st);
}

int simt_pass(int pass, const FhobProblem& p, cudaStream_t st) {
  if (p.d > 32 * DCH || head_dim_v(p) > 32 * DCH) return FHOB_ERR_SHAPE;
  if (p.dtype == FHOB_F32) return dispatch_pass<float>(pass, p, st);
  if (p.dtype == FHOB_F16) return dispatch_pass<__half>(pass, p, st);
  return dispatch_pass<__nv_bfloat16>(pass, p, st);
}

int simt_forward(const FhobProblem& p, void* o_out, float* lse_out, cudaStream_t st) {
  if (p.d > 32 * DCH || head_dim_v(p) > 32 * DCH) return FHOB_ERR_SHAPE;
  size_t smem = sizeof(float) * ((TM + 2 * TN) * pitch(p) + TM * (TN + 1));
  dim3 grid = head_grid((p.n_q + TM - 1) / TM, p.bh);
  SimtParams s = make_params(p);
  if (p.dtype == FHOB_F32) {
    FHOB_CUDA_OK(cudaFuncSetAttribute(simt_forward_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
    simt_forward_kernel<float><<<grid, NT, smem, st>>>(s, o_out, lse_out);
  } else if (p.dtype == FHOB_F16) {
    FHOB_CUDA_OK(cudaFuncSetAttribute(simt_forward_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
    simt_forward_kernel<__half><<<grid, NT, smem, st>>>(s, o_out, lse_out);
  } else {
    FHOB_CUDA_OK(cudaFuncSetAttribute(simt_forward_kernel<__nv_bfloat16>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    simt_forward_kernel<__nv_bfloat16><<<grid, NT, smem, st>>>(s, o_out, lse_out);
  }
  FHOB_CUDA_OK(cudaGetLastError());
  return FHOB_OK;
}

}  // namespace fhob
