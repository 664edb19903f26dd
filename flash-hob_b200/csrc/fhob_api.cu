// C ABI of libfhob.so: argument validation, the row-statistics pre-pass and
// dispatch of the four recomputation passes to the tensor-core or CUDA-core
// kernels.  Host wrapper role of flash_bwdbwd in the reference
// (fhog/triton_bwdbwd.py:557-648).
#include <cstdio>
#include <cstring>
#include <mutex>

#include "fhob_common.cuh"

namespace fhob {

namespace {
thread_local char g_cuda_error[512] = "";
}

void set_cuda_error(cudaError_t e, const char* where) {
  std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%s)", where, cudaGetErrorName(e),
                cudaGetErrorString(e));
}
void set_cuda_error_text(const char* text) { std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s", text); }

namespace {

// A group of `lanes` lanes (a power of two; 16 bytes of the row per lane, which covers a row of up to
// 128 elements) takes kPrepassRows query rows of one head, their loads all issued before the sums:
// D = sum_d dO*O, stored as k1 = -D, and nlc = -L*log2(e).
// Block 0 also clears the status word, so every operator call starts clean.
constexpr int kPrepassRows = 4;
template <typename T>
__global__ void prepass_kernel(const T* __restrict__ o, const T* __restrict__ d_o, const float* __restrict__ lse,
                               float* __restrict__ nlc, float* __restrict__ k1, int* status, unsigned blocks_per_head, int d,
                               int n_q, int first_live_query, View vo, View vdo, long long lse_head,
                               long long lse_batch, int lanes) {
  if (blockIdx.x == 0 && threadIdx.x == 0) *status = 0;
  // blocks do not straddle heads: head and row come from 32-bit arithmetic that is uniform per block
  const int groups = blockDim.x / lanes;
  const unsigned bh = blockIdx.x / blocks_per_head;
  const int q0 = static_cast<int>(blockIdx.x - bh * blocks_per_head) * groups * kPrepassRows + static_cast<int>(threadIdx.x) / lanes;
  constexpr int V = 16 / sizeof(T);
  const int c = (threadIdx.x & (lanes - 1)) * V;
  // the inputs may be views (strides per row / head / batch entry), the row vectors are padded per head
  const unsigned hb = bh / static_cast<unsigned>(vo.heads), hh = bh - hb * static_cast<unsigned>(vo.heads);
  const T* po = o + static_cast<long long>(hb) * vo.batch + static_cast<long long>(hh) * vo.head + c;
  const T* pd = d_o + static_cast<long long>(hb) * vdo.batch + static_cast<long long>(hh) * vdo.head + c;
  // a query the causal mask leaves without any visible key (n_k < n_q): every P of its row is
  // masked to zero in the passes, so the row contributes nothing and its dQ2 and ddO are zero.
  // Its saved L (-inf) and O (0 or NaN, depending on who produced them) are not looked at.
  uint4 a[kPrepassRows], b[kPrepassRows];
#pragma unroll
  for (int r = 0; r < kPrepassRows; ++r) {
    const int qi = q0 + r * groups;
    a[r] = b[r] = make_uint4(0u, 0u, 0u, 0u);
    if (o != nullptr && c < d && qi < n_q && qi >= first_live_query) {
      a[r] = *reinterpret_cast<const uint4*>(po + qi * vo.row);
      b[r] = *reinterpret_cast<const uint4*>(pd + qi * vdo.row);
    }
  }
  float* nlc_head = nlc + static_cast<long>(bh) * row_stride(n_q);
  float* k1_head = k1 + static_cast<long>(bh) * row_stride(n_q);
  const float* lse_h = lse + static_cast<long long>(hb) * lse_batch + static_cast<long long>(hh) * lse_head;
#pragma unroll
  for (int r = 0; r < kPrepassRows; ++r) {
    const int qi = q0 + r * groups;
    const T* ea = reinterpret_cast<const T*>(&a[r]);
    const T* eb = reinterpret_cast<const T*>(&b[r]);
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < V; ++e) acc = fmaf(static_cast<float>(ea[e]), static_cast<float>(eb[e]), acc);
    for (int off = lanes >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (c != 0 || qi >= n_q) continue;
    if (qi < first_live_query) {
      nlc_head[qi] = 0.f;
      k1_head[qi] = 0.f;
      continue;
    }
    nlc_head[qi] = -lse_h[qi] * kLog2e;
    // no O: D comes out of the sweep that yields dd and b (sum_j P dP), which then writes k1
    if (o != nullptr) k1_head[qi] = -acc;
  }
}

__global__ void row_stats_kernel(const float* k1, const float* ndd, const float* k23, float* d_out, float* dd_out,
                                 float* b_out, long rows, int n_q) {
  long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows) return;
  const long v = (i / n_q) * row_stride(n_q) + i % n_q;  // padded per head inside, dense outside
  if (d_out) d_out[i] = -k1[v];
  if (dd_out) dd_out[i] = -ndd[v];
  if (b_out) b_out[i] = -(k23[v] + k1[v] * ndd[v]);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Status word of the library itself: receives the device-side conditions of fhob_forward calls
// that pass no workspace.  In host code the symbol is a handle, not a device address, so the
// address each device gave it is looked up once, with that device current.
__device__ int g_own_status;
constexpr int kMaxDevices = 64;
std::mutex g_own_status_mutex;
int* g_own_status_ptr[kMaxDevices] = {};

int own_status_word(int** out) {
  int dev = -1;
  FHOB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return FHOB_ERR_ARG;
  std::lock_guard<std::mutex> lock(g_own_status_mutex);
  if (!g_own_status_ptr[dev]) {
    void* ptr = nullptr;
    FHOB_CUDA_OK(cudaGetSymbolAddress(&ptr, g_own_status));
    g_own_status_ptr[dev] = static_cast<int*>(ptr);
  }
  *out = g_own_status_ptr[dev];
  return FHOB_OK;
}

// strides of the first `count` matrices of a layout (those given): positive rows, everything 16-byte aligned
bool layout_ok(const FhobLayout& l, const void* const* mats, int count, size_t es) {
  const long long align = 16 / static_cast<long long>(es);
  for (int i = 0; i < count; ++i) {
    if (!mats[i]) continue;
    if (l.row[i] <= 0 || l.row[i] % align || l.head[i] % align || l.batch[i] % align || l.head[i] < 0 || l.batch[i] < 0)
      return false;
  }
  return l.lse_head >= 0 && l.lse_batch >= 0;
}

// `o_optional`: the caller may leave p->o NULL (D is then taken from sum_j P dP inside the sweep
// that yields dd and b, which only the tensor-core path does)
int validate(const FhobProblem* p, bool need_outputs, bool need_cotangents = true, bool o_optional = false) {
  if (!p) return FHOB_ERR_ARG;
  if (p->bh <= 0 || p->n_q <= 0 || p->n_k <= 0 || p->d <= 0) return FHOB_ERR_ARG;
  if (p->dtype != FHOB_BF16 && p->dtype != FHOB_F32 && p->dtype != FHOB_F16) return FHOB_ERR_ARG;
  if (p->impl != FHOB_IMPL_AUTO && p->impl != FHOB_IMPL_SIMT && p->impl != FHOB_IMPL_TCGEN05) return FHOB_ERR_ARG;
  if (p->causal != 0 && p->causal != 1) return FHOB_ERR_ARG;
  if (p->window < 0 || (p->window > 0 && !p->causal) || p->d_v < 0) return FHOB_ERR_ARG;
  const void* ins[] = {p->q, p->k, p->v, p->o, p->d_o, p->lse, p->ddq, p->ddk, p->ddv};
  for (int i = 0; i < (need_cotangents ? 9 : 6); ++i) {
    if (i == 3 && !ins[i] && o_optional && p->impl != FHOB_IMPL_SIMT && tc_supported(*p)) continue;
    if (!ins[i]) return FHOB_ERR_ARG;
    if (!aligned16(ins[i])) return FHOB_ERR_ALIGN;
  }
  if (need_outputs) {
    const void* outs[] = {p->dq2, p->dk2, p->dv2, p->ddo};
    for (const void* x : outs) {
      if (!x) return FHOB_ERR_ARG;
      if (!aligned16(x)) return FHOB_ERR_ALIGN;
    }
  }
  const size_t es = p->dtype == FHOB_F32 ? 4 : 2;
  const int dv = head_dim_v(*p);
  if ((p->d * es) % 16 != 0 || (dv * es) % 16 != 0) return FHOB_ERR_SHAPE;  // rows must stay 16-byte aligned
  if (p->d > 128 || dv > 128) return FHOB_ERR_SHAPE;
  if (!p->workspace || (reinterpret_cast<uintptr_t>(p->workspace) & 255u)) return FHOB_ERR_WORKSPACE;
  if (p->workspace_bytes < fhob_workspace_bytes(p->bh, p->n_q)) return FHOB_ERR_WORKSPACE;
  if (p->layout) {
    // views are read through tensor maps: tensor-core kernels only, strides that keep rows 16-byte aligned
    const FhobLayout& l = *p->layout;
    if (l.heads <= 0 || p->bh % l.heads != 0 || l.reserved != 0) return FHOB_ERR_ARG;
    if (p->impl == FHOB_IMPL_SIMT || !tc_supported(*p)) return FHOB_ERR_SHAPE;
    const void* mats[8] = {p->q, p->k, p->v, p->o, p->d_o, p->ddq, p->ddk, p->ddv};   // index order of FhobLayout
    if (!layout_ok(l, mats, need_cotangents ? 8 : 5, es)) return FHOB_ERR_ALIGN;
  }
  if (p->impl == FHOB_IMPL_TCGEN05 && !tc_supported(*p)) {
    // fp32 with both head dims 64 runs on the tensor cores if the workspace also holds the bf16 hi/lo copies
    if (split_dims_ok(*p)) return FHOB_ERR_WORKSPACE;
    return FHOB_ERR_SHAPE;
  }
  return FHOB_OK;
}

bool use_tc(const FhobProblem& p) {
  if (p.impl == FHOB_IMPL_SIMT) return false;
  if (p.impl == FHOB_IMPL_TCGEN05) return true;
  return tc_supported(p);
}

int run_pass(int pass, const FhobProblem* p, void* stream) {
  int st = validate(p, pass >= 3);
  if (st != FHOB_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return use_tc(*p) ? tc_pass(pass, *p, s) : simt_pass(pass, *p, s);
}

}  // namespace
}  // namespace fhob

using namespace fhob;

extern "C" {

int fhob_version(void) { return 200; }

const char* fhob_strerror(int status) {
  switch (status) {
    case FHOB_OK: return "ok";
    case FHOB_ERR_ARG: return "invalid argument (null pointer, bad dtype/impl/causal flag or non-positive size)";
    case FHOB_ERR_SHAPE: return "shape not supported (head dims must keep rows 16-byte aligned and be <= 128; "
                                "the tensor-core kernels need 16-bit elements, or fp32 with both head dims 64)";
    case FHOB_ERR_ALIGN: return "a tensor pointer is not 16-byte aligned";
    case FHOB_ERR_WORKSPACE: return "workspace missing, misaligned (256 B) or smaller than fhob_workspace_bytes() "
                                    "(fp32 on the tensor cores: smaller than fhob_workspace_bytes_problem())";
    case FHOB_ERR_CUDA: return "a CUDA call failed (see fhob_last_cuda_error)";
    case FHOB_ERR_ARCH: return "the tensor-core kernels need a compute capability 10.x device";
    case FHOB_ERR_STATIC_LIMIT: return "bh*n_q exceeds FHOB_STATIC_SCRATCH_MAX_ROWS, the capacity of the built-in "
                                       "scratch array (use fhob_bwdbwd with a caller workspace)";
    default: break;
  }
  if (status & FHOB_ERR_TIMEOUT) return "device: a bounded wait ran out of iterations (results are invalid)";
  if (status & FHOB_ERR_SMEM_ALIGN) return "device: shared memory base not 1024-byte aligned";
  if (status & FHOB_ERR_TMEM_BASE) return "device: tensor memory allocation did not start at column 0 (results are invalid)";
  return "unknown status";
}

const char* fhob_last_cuda_error(void) { return g_cuda_error; }

size_t fhob_workspace_bytes_problem(const FhobProblem* p) {
  if (!p || p->bh <= 0 || p->n_q <= 0 || p->n_k <= 0) return 0;
  if (p->impl != FHOB_IMPL_SIMT && split_dims_ok(*p)) return split_workspace_bytes(*p);
  return fhob_workspace_bytes(p->bh, p->n_q);
}

size_t fhob_workspace_bytes(int32_t bh, int32_t n_q) {
  if (bh <= 0 || n_q <= 0) return 0;
  size_t rows = static_cast<size_t>(bh) * static_cast<size_t>(row_stride(n_q));
  // the tail pad lets the key-tiled pass read whole 64-query groups of the last head
  return kWorkspaceHeaderBytes + 4 * rows * sizeof(float) + kWorkspaceTailBytes;
}

// `for_operator`: the passes of the double backward follow (not the first backward), so an fp32
// problem headed for the tensor cores also gets its bf16 hi/lo copies made here
static int run_prepass(const FhobProblem* p, void* stream, bool for_operator = true) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (for_operator && p->dtype == FHOB_F32 && use_tc(*p)) {
    int st = tc_split_inputs(*p, s);
    if (st != FHOB_OK) return st;
  }
  RowVectors rv = row_vectors(*p);
  const int dv_ = head_dim_v(*p);
  // lanes per row: enough 16-byte pieces to cover a row in one step, at most a warp
  const int pieces = dv_ * (p->dtype == FHOB_F32 ? 4 : 2) / 16;
  int lanes = 1;
  while (lanes < pieces && lanes < 32) lanes <<= 1;
  const int threads = 256, per_block = threads / lanes * kPrepassRows;
  const unsigned blocks_per_head = static_cast<unsigned>((p->n_q + per_block - 1) / per_block);
  const unsigned long long blocks = static_cast<unsigned long long>(blocks_per_head) * static_cast<unsigned>(p->bh);
  if (blocks > 0x7fffffffull) return FHOB_ERR_SHAPE;
  const unsigned grid = static_cast<unsigned>(blocks);
  // bottom-right aligned causal mask: query i sees key 0 only if i + n_k - n_q >= 0
  const int first_live = (p->causal && p->n_q > p->n_k) ? p->n_q - p->n_k : 0;
  const View vo = tensor_view(*p, kTenO, p->n_q, dv_), vdo = tensor_view(*p, kTenDO, p->n_q, dv_);
  const long long lse_head = p->layout ? p->layout->lse_head : p->n_q;
  const long long lse_batch = p->layout ? p->layout->lse_batch : static_cast<long long>(p->bh) * p->n_q;
  if (p->dtype == FHOB_BF16) {
    prepass_kernel<__nv_bfloat16><<<grid, threads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(p->o), static_cast<const __nv_bfloat16*>(p->d_o), p->lse, rv.nlc, rv.k1,
        rv.status, blocks_per_head, dv_, p->n_q, first_live, vo, vdo, lse_head, lse_batch, lanes);
  } else if (p->dtype == FHOB_F16) {
    prepass_kernel<__half><<<grid, threads, 0, s>>>(static_cast<const __half*>(p->o),
                                                       static_cast<const __half*>(p->d_o), p->lse, rv.nlc, rv.k1,
                                                       rv.status, blocks_per_head, dv_, p->n_q, first_live, vo, vdo, lse_head, lse_batch, lanes);
  } else {
    prepass_kernel<float><<<grid, threads, 0, s>>>(static_cast<const float*>(p->o),
                                                      static_cast<const float*>(p->d_o), p->lse, rv.nlc, rv.k1,
                                                      rv.status, blocks_per_head, dv_, p->n_q, first_live, vo, vdo, lse_head, lse_batch, lanes);
  }
  FHOB_CUDA_OK(cudaGetLastError());
  return FHOB_OK;
}

int fhob_prepass(const FhobProblem* p, void* stream) {
  int st = validate(p, false, true, true);
  if (st != FHOB_OK) return st;
  return run_prepass(p, stream);
}

int fhob_pass1(const FhobProblem* p, void* stream) { return run_pass(1, p, stream); }
int fhob_pass2(const FhobProblem* p, void* stream) { return run_pass(2, p, stream); }
int fhob_pass12(const FhobProblem* p, void* stream) {
  int st = validate(p, false, true, true);
  if (st != FHOB_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (use_tc(*p)) return tc_pass(p->o ? 12 : 13, *p, s);
  st = simt_pass(1, *p, s);
  return st != FHOB_OK ? st : simt_pass(2, *p, s);
}
int fhob_pass3(const FhobProblem* p, void* stream) { return run_pass(3, p, stream); }
int fhob_pass4(const FhobProblem* p, void* stream) { return run_pass(4, p, stream); }

int fhob_bwdbwd(const FhobProblem* p, void* stream) {
  int st = validate(p, true, true, true);
  if (st != FHOB_OK) return st;
  st = run_prepass(p, stream);
  if (st != FHOB_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (use_tc(*p)) {
    // dd and b come out of one sweep (sum_j P dP = D makes b linear in sums that need no dd)
    const int kPasses[3] = {p->o ? 12 : 13, 3, 4};
    for (int pass : kPasses) {
      st = tc_pass(pass, *p, s);
      if (st != FHOB_OK) return st;
    }
    return FHOB_OK;
  }
  for (int pass = 1; pass <= 4; ++pass) {
    st = simt_pass(pass, *p, s);
    if (st != FHOB_OK) return st;
  }
  return FHOB_OK;
}

int fhob_row_stats(const FhobProblem* p, float* d_out, float* dd_out, float* b_out, void* stream) {
  int st = validate(p, false, true, true);
  if (st != FHOB_OK) return st;
  RowVectors rv = row_vectors(*p);
  long rows = static_cast<long>(p->bh) * p->n_q;
  unsigned grid = static_cast<unsigned>((rows + 255) / 256);
  row_stats_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(rv.k1, rv.ndd, rv.k23, d_out, dd_out, b_out,
                                                                        rows, p->n_q);
  FHOB_CUDA_OK(cudaGetLastError());
  return FHOB_OK;
}

int fhob_read_status(const FhobProblem* p, void* stream) {
  if (!p) return FHOB_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const void* word = p->workspace;
  if (!word) {
    // no workspace: the library's own word, which fhob_forward uses in that case
    int* own = nullptr;
    int st = own_status_word(&own);
    if (st != FHOB_OK) return st;
    word = own;
  }
  int host = 0;
  FHOB_CUDA_OK(cudaMemcpyAsync(&host, word, sizeof(int), cudaMemcpyDeviceToHost, s));
  FHOB_CUDA_OK(cudaStreamSynchronize(s));
  return host;
}

int fhob_visible_tiles(int q_stationary, int m0, int rows, int tile, int n_q, int n_k, int causal, int window,
                       int* t_begin, int* t_end) {
  if (!t_begin || !t_end || rows <= 0 || tile <= 0 || n_q <= 0 || n_k <= 0 || m0 < 0 || window < 0) return FHOB_ERR_ARG;
  visible_tiles(q_stationary != 0, m0, rows, tile, q_stationary ? n_k : n_q, n_k - n_q, causal, window, *t_begin,
                *t_end);
  return FHOB_OK;
}

int fhob_selftest_expired_wait(void* workspace, size_t workspace_bytes, void* stream) {
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < sizeof(int))
    return FHOB_ERR_WORKSPACE;
  return tc_selftest_expired_wait(static_cast<int*>(workspace), static_cast<cudaStream_t>(stream));
}

int fhob_forward(const FhobProblem* p, void* o_out, float* lse_out, void* stream) {
  if (!p || !p->q || !p->k || !p->v || !lse_out) return FHOB_ERR_ARG;
  if (p->bh <= 0 || p->n_q <= 0 || p->n_k <= 0 || p->d <= 0 || p->d > 128 || p->d_v < 0 || p->d_v > 128)
    return FHOB_ERR_SHAPE;
  if (p->dtype != FHOB_BF16 && p->dtype != FHOB_F32 && p->dtype != FHOB_F16) return FHOB_ERR_ARG;
  if (p->window < 0 || (p->window > 0 && p->causal != 1)) return FHOB_ERR_ARG;
  if (p->impl != FHOB_IMPL_AUTO && p->impl != FHOB_IMPL_SIMT && p->impl != FHOB_IMPL_TCGEN05) return FHOB_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool tc_ok = aligned16(p->q) && aligned16(p->k) && aligned16(p->v) && aligned16(o_out) &&
                     tc_first_order_supported(*p);
  if (p->layout) {
    // views of q, k, v: tensor-core kernels only
    const FhobLayout& l = *p->layout;
    if (l.heads <= 0 || p->bh % l.heads != 0 || l.reserved != 0) return FHOB_ERR_ARG;
    if (p->impl == FHOB_IMPL_SIMT || !tc_ok) return FHOB_ERR_SHAPE;
    const void* mats[3] = {p->q, p->k, p->v};
    if (!layout_ok(l, mats, 3, p->dtype == FHOB_F32 ? 4 : 2)) return FHOB_ERR_ALIGN;
  }
  if (p->impl == FHOB_IMPL_TCGEN05 && !tc_ok) return FHOB_ERR_SHAPE;
  if (p->impl != FHOB_IMPL_SIMT && tc_ok) {
    int* status = static_cast<int*>(p->workspace);
    if (status) {
      if ((reinterpret_cast<uintptr_t>(p->workspace) & 255u) || p->workspace_bytes < sizeof(int)) return FHOB_ERR_WORKSPACE;
    } else {
      int st = own_status_word(&status);
      if (st != FHOB_OK) return st;
    }
    FHOB_CUDA_OK(cudaMemsetAsync(status, 0, sizeof(int), s));  // every call starts with a clean status word
    return tc_forward(*p, o_out, lse_out, status, s);
  }
  return simt_forward(*p, o_out, lse_out, s);
}

int fhob_backward(const FhobProblem* p, void* dq, void* dk, void* dv, void* stream) {
  if (!dq || !dk || !dv) return FHOB_ERR_ARG;
  int st = validate(p, false, false);
  if (st != FHOB_OK) return st;
  if (!aligned16(dq) || !aligned16(dk) || !aligned16(dv)) return FHOB_ERR_ALIGN;
  st = run_prepass(p, stream, false);  // stores -L*log2(e) and -D in the workspace
  if (st != FHOB_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool tc = p->impl == FHOB_IMPL_TCGEN05 || (p->impl == FHOB_IMPL_AUTO && tc_first_order_supported(*p));
  return tc ? tc_backward(*p, dq, dk, dv, s) : simt_backward(*p, dq, dk, dv, s);
}

}  // extern "C"
