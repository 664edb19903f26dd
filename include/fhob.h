/*
 * fhob.h — C ABI of the B200 double-backward flash attention library (libfhob.so).
 *
 * The library replaces one operator of the reference project: the double
 * backward of scaled-dot-product attention,
 *
 *     flash_bwdbwd(Q, K, V, O, dO, ddQ, ddK, ddV, L, scale) -> (dQ2, dK2, dV2, ddO)
 *
 * (reference: fhog/triton_bwdbwd.py:557-648, exported at fhog/__init__.py:1-3).
 * Every entry point takes plain device pointers and sizes, launches on the
 * CUDA stream it is given and returns an int status (0 = ok).  No entry point
 * allocates device memory unless its comment says so; scratch is a caller
 * provided workspace of fhob_workspace_bytes() bytes.
 *
 * Layout: every matrix is row-major (BH, N, D) with the batch and head axes
 * folded into BH like the reference does (fhog/triton_bwdbwd.py:577), rows
 * contiguous and 16-byte aligned.  L is fp32 (BH, N_Q).
 */
#ifndef FHOB_H_
#define FHOB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types of the eleven matrices (all share one type). */
/* FHOB_F16: the reference's benchmark dtype (fhog/benchhhh.py:19); tensor-core path like bf16 */
enum { FHOB_BF16 = 0, FHOB_F32 = 1, FHOB_F16 = 2 };

/* Kernel families.  AUTO = tcgen05/TMEM/TMA tensor-core kernels for 16-bit
 * elements (head dims up to 128, multiples of 8) and for fp32 with both head dims at most 64 when the
 * workspace has fhob_workspace_bytes_problem() bytes; CUDA-core kernels for
 * everything else.  SIMT forces the CUDA-core kernels for any type
 * (debugging aid; same four passes, same row statistics). */
enum { FHOB_IMPL_AUTO = 0, FHOB_IMPL_SIMT = 1, FHOB_IMPL_TCGEN05 = 2 };

/* Status codes.  Device-side conditions are accumulated (OR-ed) into the
 * status word at the start of the workspace and fetched with
 * fhob_read_status(). */
enum {
  FHOB_OK = 0,
  FHOB_ERR_ARG = 1,        /* null pointer, bad dtype/impl, non-positive size */
  FHOB_ERR_SHAPE = 2,      /* head dim / sequence length not supported by the chosen kernels */
  FHOB_ERR_ALIGN = 3,      /* a pointer is not 16-byte aligned */
  FHOB_ERR_WORKSPACE = 4,  /* workspace missing or too small */
  FHOB_ERR_CUDA = 5,       /* a CUDA runtime/driver call failed (see fhob_last_cuda_error) */
  FHOB_ERR_ARCH = 6,       /* tensor-core kernels need compute capability 10.x */
  FHOB_ERR_STATIC_LIMIT = 7, /* fhob_bwdbwd_static_scratch: bh*n_q exceeds FHOB_STATIC_SCRATCH_MAX_ROWS */
  FHOB_ERR_TIMEOUT = 64,   /* device: a bounded mbarrier wait ran out (bit in the status word) */
  FHOB_ERR_SMEM_ALIGN = 128, /* device: dynamic shared memory base was not 1024-byte aligned */
  FHOB_ERR_TMEM_BASE = 256   /* device: the tensor-memory allocation did not start at column 0 */
};

/*
 * Optional memory layout of the eight matrices and of lse, for callers whose
 * tensors are views (a (B, N, H, D) projection seen as (B, H, N, D), a slice
 * of a fused QKV tensor, ...).  The reference passes the strides of every
 * tensor to its kernels (fhog/triton_bwdbwd.py:594-610, :628-640); this is the
 * same information.  Strides are in elements; the last dim (d) is contiguous.
 * Head bh of the folded axis is (batch b, head h) = (bh / heads, bh % heads).
 * Index order of the arrays: q, k, v, o, d_o, ddq, ddk, ddv.
 * Only the tensor-core kernels take a layout (impl AUTO resolving to them, or
 * TCGEN05); every stride must keep rows 16-byte aligned.  Results are always
 * written contiguous (bh, n, d).
 */
typedef struct FhobLayout {
  int32_t heads;       /* heads per batch entry; bh must be a multiple of it */
  int32_t reserved;    /* must be 0 */
  int64_t row[8];      /* stride between consecutive rows of a head */
  int64_t head[8];     /* stride between the heads of one batch entry */
  int64_t batch[8];    /* stride between batch entries */
  int64_t lse_head;    /* lse (rows contiguous): stride between heads ... */
  int64_t lse_batch;   /* ... and between batch entries */
} FhobLayout;

/*
 * One double-backward problem.  Replaces the argument list of
 * flash_bwdbwd (fhog/triton_bwdbwd.py:558) and of its two kernel launches
 * (fhog/triton_bwdbwd.py:586-612, :620-646).
 */
typedef struct FhobProblem {
  int32_t bh;      /* folded batch*heads */
  int32_t n_q;     /* query rows per head */
  int32_t n_k;     /* key rows per head */
  int32_t d;       /* head dim of q, k, ddq, ddk, dq2, dk2 (and of the v side too when d_v is 0, like the
                      reference, which has a single D: :577) */
  int32_t dtype;   /* FHOB_BF16, FHOB_F16 or FHOB_F32 */
  int32_t causal;  /* 0, or 1 = bottom-right aligned causal mask: key j visible to query i iff i + n_k - n_q >= j.
                      With n_k < n_q the first n_q - n_k queries see no key at all: their dQ2 and ddO rows are
                      zero, they add nothing to dK2 and dV2, and their lse / o entries are not read
                      (fhob_forward writes lse = -inf and o = 0 there) */
  int32_t impl;    /* FHOB_IMPL_* */
  float scale;     /* softmax scale */
  int32_t window;  /* sliding_window_length of jax_refs/flash_impl.py:86-91: 0 = none; W > 0 (needs causal = 1)
                      additionally hides keys with (i + n_k - n_q) - j >= W */
  int32_t d_v;     /* head dim of v, ddv, o, d_o, ddo, dv2 when it differs from d (the reference's maths allows
                      two head dims, jax_refs/flash_impl.py:381-389); 0 = same as d */
  /* inputs, device pointers */
  const void* q;   /* (bh, n_q, d) */
  const void* k;   /* (bh, n_k, d) */
  const void* v;   /* (bh, n_k, d_v) */
  const void* o;   /* (bh, n_q, d_v) forward output; may be NULL for fhob_bwdbwd / fhob_pass12 on the tensor-core
                      path: D = rowsum(dO * O) (reference :580) is then replaced by the equal sum_j P dP */
  const void* d_o; /* (bh, n_q, d_v) cotangent of o in the first backward */
  const void* ddq; /* (bh, n_q, d) cotangent of dQ */
  const void* ddk; /* (bh, n_k, d) cotangent of dK */
  const void* ddv; /* (bh, n_k, d_v) cotangent of dV */
  const float* lse; /* (bh, n_q) fp32 logsumexp of the masked scaled scores */
  /* outputs, device pointers, same element type as the inputs */
  void* dq2; /* (bh, n_q, d) */
  void* dk2; /* (bh, n_k, d) */
  void* dv2; /* (bh, n_k, d_v) */
  void* ddo; /* (bh, n_q, d_v) */
  /* scratch: fhob_workspace_bytes(bh, n_q) bytes, 256-byte aligned */
  void* workspace;
  size_t workspace_bytes;
  /* NULL = every matrix contiguous (bh, n, d) and lse contiguous (bh, n_q); see FhobLayout */
  const struct FhobLayout* layout;
} FhobProblem;

/* Library version (major*10000 + minor*100 + patch). */
int fhob_version(void);

/* Text for a status code. */
const char* fhob_strerror(int status);

/* Text of the last CUDA error this thread's calls ran into ("" if none). */
const char* fhob_last_cuda_error(void);

/*
 * Bytes of scratch one problem needs: a 256-byte header holding the device
 * status word plus four fp32 row vectors (-L*log2e, -D, -dd, -D*dd - b) of
 * bh * ceil4(n_q) entries: each head's slice is padded to a multiple of four
 * so that it starts on a 16-byte boundary.  This is the whole extra memory of the operator —
 * linear in n_q.  Replaces the reference's D, dD and B temporaries
 * (fhog/triton_bwdbwd.py:580-584).
 */
size_t fhob_workspace_bytes(int32_t bh, int32_t n_q);

/*
 * Bytes of scratch that let the library take its fastest path for this
 * particular problem (reads bh, n_q, n_k, d, d_v, dtype, impl).  Equal to
 * fhob_workspace_bytes(bh, n_q) except for fp32 problems with both head dims
 * at most 64 (multiples of 4): those run on the tensor cores (every fp32 operand as a bf16 hi + lo
 * pair, three products per contraction, fp32 accumulation) if the workspace
 * also has room for the bf16 copies of the seven inputs (their size again:
 * still linear in the sequence lengths).  With a smaller workspace such a
 * problem runs on the CUDA-core kernels (impl AUTO) or is refused with
 * FHOB_ERR_WORKSPACE (impl TCGEN05).  The reference has no counterpart: its
 * Triton kernels take whatever precision tl.dot gives fp32 inputs.
 */
size_t fhob_workspace_bytes_problem(const FhobProblem* p);

/*
 * The whole operator: row-statistics pre-pass and the recomputation
 * passes, queued on `stream` (a cudaStream_t) without synchronising.
 * Replaces flash_bwdbwd (fhog/triton_bwdbwd.py:557-648).
 */
int fhob_bwdbwd(const FhobProblem* p, void* stream);

/*
 * The single stages, for unit tests and profiling.  They must run in this
 * order on one stream because each consumes row vectors the previous wrote.
 *
 * fhob_prepass: clears the status word, D_i = sum_d dO*O (reference :580),
 *               stores -D*scale and -L*log2(e).
 * fhob_pass1:   dd_i = sum_j ddS_ij P_ij                 (reference :178-215)
 * fhob_pass2:   b_i  = sum_j dP2_ij P_ij                 (reference :217-255)
 * fhob_pass3:   dQ2 and ddO                              (reference :257-313)
 * fhob_pass4:   dK2 and dV2, key-tiled                   (reference :321-535)
 */
int fhob_prepass(const FhobProblem* p, void* stream);
int fhob_pass1(const FhobProblem* p, void* stream);
int fhob_pass2(const FhobProblem* p, void* stream);
int fhob_pass3(const FhobProblem* p, void* stream);
int fhob_pass4(const FhobProblem* p, void* stream);

/*
 * dd and b in one sweep over the keys; equivalent to fhob_pass1 followed by
 * fhob_pass2 and what fhob_bwdbwd runs on the tensor-core path.  With
 * sum_j P_ij dP_ij = D_i the reference's b (:236-243) is
 *   b_i = sum_j P_ij (X_ij + dP_ij ddS_ij) - 2 D_i dd_i,
 * whose sums do not need dd_i while the tiles stream by, so S, P and ddS
 * are recomputed once instead of twice (5 contractions instead of 3 + 5).
 * The reference has no such stage.  (The CUDA-core path runs its two passes.)
 */
int fhob_pass12(const FhobProblem* p, void* stream);

/*
 * Copies the row statistics out of the workspace into caller device buffers
 * of bh*n_q floats each, undoing the internal sign/scale folding:
 * d_out = D, dd_out = dd, b_out = b.  Any of the three may be NULL.
 * (The reference keeps these as the tensors D, dD, B: :580-584.)
 */
int fhob_row_stats(const FhobProblem* p, float* d_out, float* dd_out, float* b_out, void* stream);

/*
 * Synchronises `stream`, reads the device status word of the workspace and
 * returns it (0 = every bounded wait completed).  With p->workspace NULL it
 * reads the library's own per-device word instead, which is where
 * fhob_forward reports when it is given no workspace.  The reference has no
 * counterpart; its kernels cannot time out.
 */
int fhob_read_status(const FhobProblem* p, void* stream);

/*
 * The tile-range rule every kernel of the library uses (host evaluation, no
 * GPU needed): for stationary rows [m0, m0 + rows) — queries if q_stationary,
 * else keys — the half-open range [*t_begin, *t_end) of streamed tiles of
 * `tile` rows that can hold a pair visible under the mask of
 * jax_refs/flash_impl.py:86-91 (causal, bottom-right aligned, optional
 * sliding window).  Exposed so that the rule can be checked exhaustively
 * against the mask definition; the reference has no counterpart (its
 * kernels visit every tile).
 */
int fhob_visible_tiles(int q_stationary, int m0, int rows, int tile, int n_q, int n_k, int causal, int window,
                       int* t_begin, int* t_end);

/*
 * Self-test of the bounded device waits.  Queues one warp whose only wait is
 * on an mbarrier nothing ever arrives on; after about a second the wait gives
 * up, ORs FHOB_ERR_TIMEOUT into the status word at the start of `workspace`
 * (256-byte aligned device memory) and the kernel returns normally, so the
 * context stays usable.  This is the path every kernel of the library takes
 * when a wait runs out; fhob_read_status then reports it.  The reference has
 * no counterpart.
 */
int fhob_selftest_expired_wait(void* workspace, size_t workspace_bytes, void* stream);

/*
 * O(N)-memory producer of the two saved forward results the operator
 * consumes: O = softmax(QK^T scale) V in the input element type and the fp32
 * logsumexp L.  Role of flash_kernel / produce_L in the reference
 * (fhog/triton_flash.py:12-133, :252-258), which is dense, rounds L to the
 * input type and refuses causal masks.  Uses p->q, k, v, scale, causal,
 * window, impl; writes `o_out` (bh, n_q, d) and `lse_out` (bh, n_q).
 * `o_out` may be NULL when only the logsumexp is wanted (the role of
 * produce_L): the P V product is then skipped altogether.
 * 16-bit inputs with head dims up to 128 (multiples of 8; d_v may differ from d) and fp32
 * inputs with both head dims at most 64 and a workspace of
 * fhob_workspace_bytes_problem() bytes (split bf16 operands) run on the tensor
 * cores (impl AUTO or TCGEN05), everything else on CUDA cores.  Device-side conditions (a wait
 * that ran out) go to the status word at the start of p->workspace, or, when
 * p->workspace is NULL, to a word the library keeps per device; either is
 * cleared by the call and read with fhob_read_status(p, stream).
 */
int fhob_forward(const FhobProblem* p, void* o_out, float* lse_out, void* stream);

/*
 * First backward of attention from the saved forward results, O(N) memory:
 * dQ, dK, dV from q, k, v, o, d_o, lse (scale, causal) of `p`; the other
 * cotangent pointers of `p` are ignored, the workspace is used (and
 * overwritten).  Role of FlashAttention2.backward / flash_backward_torch in
 * the reference (fhog/triton_flash.py:190-220), which materialises S, P, dP,
 * dS.  It is the function whose derivative fhob_bwdbwd computes
 * (jax_refs/flash_impl.py:124-173).  Tensor cores or CUDA cores as for
 * fhob_forward.
 */
int fhob_backward(const FhobProblem* p, void* dq, void* dk, void* dv, void* stream);

/*
 * The operator for callers that cannot allocate device memory at all.
 * (No counterpart in the reference, whose wrapper allocates its temporaries
 * with torch on every call.)
 *
 * Who needs it: a host that owns all device memory itself and does not let an
 * operator call cudaMalloc - an engine that carves everything out of one
 * arena sized at start-up, a plug-in running inside another framework's
 * memory plan, a latency-bound loop where an allocation could synchronise the
 * device - and that has no spare buffer to lend as the workspace either.
 * Same arguments and results as fhob_bwdbwd, except that p->workspace and
 * p->workspace_bytes are ignored: the status word and the four row vectors
 * live in a fixed device array inside the library (about 4 MiB, held on every
 * GPU that loads the library until the process exits).  The call performs no
 * cudaMalloc/cudaFree and calls no allocating library routine.
 *
 * Limit: bh * n_q (n_q rounded up to a multiple of four) <= FHOB_STATIC_SCRATCH_MAX_ROWS, otherwise
 * FHOB_ERR_STATIC_LIMIT is returned and nothing is launched.
 *
 * The first call on each device looks up the device address of that array
 * (one cudaGetSymbolAddress, with the calling thread's current device); make
 * that first call before starting any stream capture on that device.
 *
 * All calls on a device share the one array, which still holds the previous
 * call's row vectors; the operator clears the status word itself and writes
 * every entry before reading it, so nothing has to be reset between calls.
 * Because of the sharing, two calls whose kernels can overlap on the GPU (two
 * streams, two host threads on one device) race on the array: issue these
 * calls on one stream, or otherwise order them.  The array belongs to the
 * calling thread's current device, so make the device that holds the tensors
 * current before the call.  fhob_read_status() does not see this array; its
 * status word is read with fhob_static_scratch_status().
 */
#define FHOB_STATIC_SCRATCH_MAX_ROWS 262144
int fhob_bwdbwd_static_scratch(const FhobProblem* p, void* stream);

/*
 * Synchronises `stream` and returns the device status word of the built-in
 * scratch array on the current device (0 = every bounded wait of the last
 * fhob_bwdbwd_static_scratch call completed).  Allocates nothing.  No
 * counterpart in the reference.
 */
int fhob_static_scratch_status(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FHOB_H_ */
