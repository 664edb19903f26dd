// Shared definitions of the double-backward attention kernels.
//
// Notation (reference: fhog/triton_bwdbwd.py:178-313, jax_refs/flash_impl.py:176-229):
//   S   = Q K^T * scale            P   = exp(S - L)
//   A2  = ddQ K^T + Q ddK^T        ddS = scale * A2
//   dP  = dO V^T                   X   = dO ddV^T
//   D_i = sum_d dO O               dd_i = sum_j ddS P
//   dP2 = X + dP (ddS - dd) - D ddS      b_i = sum_j dP2 P
//   dS  = scale P (dP - D)         dS2 = scale P (dP2 - b)     ddP = P (ddS - dd)
//   dQ2 = dS ddK + dS2 K           ddO = ddP V + P ddV
//   dK2 = dS^T ddQ + dS2^T Q       dV2 = ddP^T dO
//
// Four row vectors are staged in the workspace with signs folded in so that the
// per-element work is a few FMAs (dP' = dP + k1, X' = X + k23, t = scale*A2 + ndd):
//   nlc = -L*log2(e)   k1 = -D   ndd = -dd   k23 = -D*dd - b
//   P = exp2(S_raw*scale*log2e + nlc)       ddP = P t
//   dS = (P scale) dP'                      dS2 = (P scale) (dP' t + X')
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fhob.h"

namespace fhob {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kWorkspaceHeaderBytes = 256;
constexpr int kWorkspaceTailBytes = 1024;

struct RowVectors {
  int* status;  // device status word (workspace header)
  float* nlc;   // -L * log2(e)
  float* k1;    // -D
  float* ndd;   // -dd
  float* k23;   // -D*dd - b
};

// Head dim of V, ddV, dO, O and of the results ddO, dV2 (0 in the struct = same as d).
inline int head_dim_v(const FhobProblem& p) { return p.d_v > 0 ? p.d_v : p.d; }

// Where the rows of one input matrix are: element strides between rows, between the heads of a
// batch entry and between batch entries (FhobLayout), or the contiguous (bh, n, d) default.
// Index order of FhobLayout: q, k, v, o, d_o, ddq, ddk, ddv.
enum { kTenQ = 0, kTenK = 1, kTenV = 2, kTenO = 3, kTenDO = 4, kTenDDQ = 5, kTenDDK = 6, kTenDDV = 7 };
struct View {
  int heads, batches;          // bh = batches * heads
  long long row, head, batch;  // element strides
};
inline View tensor_view(const FhobProblem& p, int which, int n_rows, int d) {
  View v;
  if (p.layout) {
    v.heads = p.layout->heads;
    v.batches = p.bh / p.layout->heads;
    v.row = p.layout->row[which];
    v.head = p.layout->head[which];
    v.batch = p.layout->batch[which];
  } else {
    v.heads = p.bh;
    v.batches = 1;
    v.row = d;
    v.head = static_cast<long long>(n_rows) * d;
    v.batch = static_cast<long long>(p.bh) * n_rows * d;
  }
  return v;
}
inline View contiguous_view(int bh, int n_rows, int d) {
  View v;
  v.heads = bh; v.batches = 1; v.row = d;
  v.head = static_cast<long long>(n_rows) * d;
  v.batch = static_cast<long long>(bh) * n_rows * d;
  return v;
}

// Entries per head of a row vector: n_q rounded up to a multiple of four, so that every head's
// slice (and every 64-query group the key-tiled kernels fetch with a bulk copy) starts on a
// 16-byte boundary whatever n_q is.
__host__ __device__ inline int row_stride(int n_q) { return (n_q + 3) & ~3; }

inline RowVectors row_vectors(const FhobProblem& p) {
  RowVectors r;
  char* base = static_cast<char*>(p.workspace);
  size_t n = static_cast<size_t>(p.bh) * static_cast<size_t>(row_stride(p.n_q));
  r.status = reinterpret_cast<int*>(base);
  float* f = reinterpret_cast<float*>(base + kWorkspaceHeaderBytes);
  r.nlc = f;
  r.k1 = f + n;
  r.ndd = f + 2 * n;
  r.k23 = f + 3 * n;
  return r;
}

// fp32 problems on the tensor cores: bf16 hi/lo copies of the seven inputs, rows of [hi(64) | lo(64)],
// stored behind the row vectors in the workspace (each copy has the bytes of its fp32 original).
struct SplitBuffers {
  void *q, *ddq, *d_o, *k, *ddk, *v, *ddv;
};
inline size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }
// head dims the split scheme takes: rows of up to 64 fp32 columns, 16-byte aligned
inline bool split_dims_ok(const FhobProblem& p) {
  const int dv = head_dim_v(p);
  return p.dtype == FHOB_F32 && p.d > 0 && p.d <= 64 && p.d % 4 == 0 && dv <= 64 && dv % 4 == 0;
}
inline size_t split_workspace_bytes(const FhobProblem& p) {
  const size_t q_bytes = align256(static_cast<size_t>(p.bh) * p.n_q * 256);
  const size_t k_bytes = align256(static_cast<size_t>(p.bh) * p.n_k * 256);
  return align256(fhob_workspace_bytes(p.bh, p.n_q)) + 3 * q_bytes + 4 * k_bytes;
}
inline SplitBuffers split_buffers(const FhobProblem& p) {
  const size_t q_bytes = align256(static_cast<size_t>(p.bh) * p.n_q * 256);
  const size_t k_bytes = align256(static_cast<size_t>(p.bh) * p.n_k * 256);
  char* b = static_cast<char*>(p.workspace) + align256(fhob_workspace_bytes(p.bh, p.n_q));
  SplitBuffers s;
  s.q = b; s.ddq = b + q_bytes; s.d_o = b + 2 * q_bytes;
  b += 3 * q_bytes;
  s.k = b; s.ddk = b + k_bytes; s.v = b + 2 * k_bytes; s.ddv = b + 3 * k_bytes;
  return s;
}

// Mask of the reference (jax_refs/flash_impl.py:86-91): with off = n_k - n_q, key j is visible to
// query i iff 0 <= i + off - j, and i + off - j < window when a sliding window is set.
__host__ __device__ inline bool pair_visible(int qi, int kj, int off, int causal, int window) {
  if (!causal) return true;
  const int dist = qi + off - kj;
  return dist >= 0 && (window <= 0 || dist < window);
}

// Range [t_begin, t_end) of streamed tiles (tn rows each, n_strm rows in all) that can hold a
// visible pair for the stationary rows [m0, m0 + tm): streamed keys when the queries are
// stationary, streamed queries when the keys are.
__host__ __device__ inline void visible_tiles(bool q_stationary, int m0, int tm, int tn, int n_strm, int off,
                                              int causal, int window, int& t_begin, int& t_end) {
  t_begin = 0;
  t_end = (n_strm + tn - 1) / tn;
  if (!causal) return;
  long first, last;  // inclusive range of streamed rows visible to any stationary row
  if (q_stationary) {
    last = static_cast<long>(m0) + tm - 1 + off;
    first = window > 0 ? static_cast<long>(m0) + off - window + 1 : 0;
  } else {
    first = static_cast<long>(m0) - off;
    last = window > 0 ? static_cast<long>(m0) + tm - 1 - off + window - 1 : static_cast<long>(n_strm) - 1;
  }
  if (last < 0) {
    t_end = 0;
  } else if (last / tn + 1 < t_end) {
    t_end = static_cast<int>(last / tn + 1);
  }
  if (first > 0) t_begin = static_cast<int>(first / tn < t_end ? first / tn : t_end);
  if (t_begin > t_end) t_begin = t_end;
}

// Per-thread record of the last CUDA error (read through fhob_last_cuda_error).
void set_cuda_error(cudaError_t e, const char* where);
void set_cuda_error_text(const char* text);

#define FHOB_CUDA_OK(expr)                                  \
  do {                                                      \
    cudaError_t e__ = (expr);                               \
    if (e__ != cudaSuccess) {                               \
      ::fhob::set_cuda_error(e__, #expr);                   \
      return FHOB_ERR_CUDA;                                 \
    }                                                       \
  } while (0)

// CUDA-core kernels (fp32 accumulate, any sizes): simt_kernels.cu
int simt_pass(int pass, const FhobProblem& p, cudaStream_t s);
int simt_forward(const FhobProblem& p, void* o_out, float* lse_out, cudaStream_t s);
int simt_backward(const FhobProblem& p, void* dq, void* dk, void* dv, cudaStream_t s);

// tcgen05 / TMEM / TMA kernels (bf16, d in {64,128}): tc_kernels.cu
bool tc_supported(const FhobProblem& p);
bool tc_split_supported(const FhobProblem& p);            // fp32 on the tensor cores (split operands)
// which inputs tc_split_inputs copies (the operator needs all seven, the forward q, k, v, ...)
enum { kSplitQ = 1, kSplitDDQ = 2, kSplitDO = 4, kSplitK = 8, kSplitDDK = 16, kSplitV = 32, kSplitDDV = 64, kSplitAll = 127 };
int tc_split_inputs(const FhobProblem& p, cudaStream_t s, int which = kSplitAll);  // writes hi/lo copies into the workspace
int tc_pass(int pass, const FhobProblem& p, cudaStream_t s);

// tensor-core forward (O, L) and first backward (dQ, dK, dV): tc_first_order.cu
bool tc_first_order_supported(const FhobProblem& p);
int tc_forward(const FhobProblem& p, void* o_out, float* lse_out, int* status, cudaStream_t s);
int tc_backward(const FhobProblem& p, void* dq, void* dk, void* dv, cudaStream_t s);
int tc_selftest_expired_wait(int* status, cudaStream_t s);

}  // namespace fhob
