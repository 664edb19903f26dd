// Pieces shared by the tensor-core kernels (sm_100a): CTA shape and warp roles, the bounded
// mbarrier wait, the K-step loops that issue tcgen05.mma for a whole tile product, and the TMA
// tensor-map builder.  Included by each .cu file that holds such kernels; everything lives in an
// unnamed namespace.
#pragma once

#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "fhob_common.cuh"
#include "sm100_ptx.cuh"

namespace fhob {
namespace {

using namespace ptx;

constexpr int BM = 128;
constexpr int EW_THREADS = 256;
constexpr int MMA_WARP = 0;   // issues the products of chain 1 (group A and the outputs it feeds); owns TMEM
constexpr int MMA_WARP2 = 1;  // issues the products of chain 2 (group B and the outputs it feeds)
constexpr int TMA_WARP = 2;
constexpr int MMA_WARP3 = 3;  // issues A2 += stat1 . strm0^T behind chain 1's stacked product
constexpr int EW_WARP0 = 4;   // elementwise warps 4..11
constexpr int NTHREADS = 384;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_LIMIT = 232448;  // 227 KB per CTA
constexpr int SMEM_TAIL = 1024;     // barriers, TMEM base, abort flag, row-sum exchange
constexpr long long kTimeoutCycles = 2000000000LL;   // about a second
constexpr long long kPeerCheckCycles = 2000000LL;    // after ~1 ms also give up if another CTA timed out

// Bounded wait on an mbarrier phase.  `b` is the CTA's barrier block (any struct with an
// `abort_flag`): a wait that runs out sets FHOB_ERR_TIMEOUT in the status word and the CTA-wide
// abort flag, and every later wait of the CTA returns false at once.
template <class B>
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, B* b, int* status) {
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

// Descriptor words of 128-byte-swizzled bf16 tiles (rows of 64 elements, 8-row groups 1024 B apart).
constexpr uint32_t kDescHi = umma_desc_hi_sw128(1024);

// D (+)= A . B^T with both tiles K-major in shared memory.  a_lo / b_lo are the low descriptor
// words of the tiles; a K=16 step advances 32 bytes inside a 64-column box, the second box of a
// D=128 tile starts A_BOX / B_BOX bytes after the first.  The number of B rows (N) is in idesc.
template <int D, int A_BOX, int B_BOX, int KS0 = 0, int KS1 = D / 16>
__device__ __forceinline__ void gemm_ss(bool leader, uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                        bool accumulate) {
#pragma unroll
  for (int ks = KS0; ks < KS1; ++ks) {
    const uint32_t a = a_lo + (((ks / 4) * A_BOX + (ks % 4) * 32) >> 4);
    const uint32_t b = b_lo + (((ks / 4) * B_BOX + (ks % 4) * 32) >> 4);
    umma_ss_split(d_tmem, a, b, kDescHi, idesc, (accumulate || ks > 0) ? 1u : 0u, leader);
  }
}

// D (+)= A . B with A = bf16 tile in TMEM (128 x BN, 8 columns per 16 rows of B) and B = streamed
// tile (BN rows x N columns, N in idesc) read MN-major: the contraction runs down the BN rows,
// 2048 bytes per step.  b_lo must carry the leading byte offset (distance between the tile's two
// 64-column boxes; not used when the tile has a single box).
template <int BN>
__device__ __forceinline__ void gemm_ts(bool leader, uint32_t d_tmem, uint32_t a_region, uint32_t b_lo,
                                        uint32_t idesc, bool accumulate) {
  constexpr int CH = BN / 32;
#pragma unroll
  for (int s = 0; s < BN / 16; ++s) {
    const uint32_t a = a_region + (s / CH) * (BN / 2) + 8 * (s % CH);
    umma_ts_split(d_tmem, a, b_lo + ((s * 2048) >> 4), kDescHi, idesc, (accumulate || s > 0) ? 1u : 0u, leader);
  }
}

__device__ __forceinline__ void load4(uint32_t smem_addr, float (&v)[4]) {
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "r"(smem_addr));
}

__device__ __forceinline__ float2 f2(uint32_t lo, uint32_t hi) {
  return make_float2(__uint_as_float(lo), __uint_as_float(hi));
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

// 16-bit matrix of `n` rows x `d` columns per head, heads and batch entries at the strides of `v`:
// a 4-D map (d, n, heads, batches), box = 64 columns x `rows` rows of one head, 128-byte swizzle.
// Encoded maps are kept in a small per-thread table: a training step calls the operator with the
// same tensors again and again, and an encode costs a few microseconds of host time per map.
struct MapKey {
  const void* base;
  int n, d, rows, f16, heads, batches;
  long long row, head, batch;
  bool operator==(const MapKey& o) const {
    return base == o.base && n == o.n && d == o.d && rows == o.rows && f16 == o.f16 && heads == o.heads &&
           batches == o.batches && row == o.row && head == o.head && batch == o.batch;
  }
};

int make_map(CUtensorMap* m, const void* base, const View& v, int n, int d, int rows, bool f16) {
  constexpr int kSlots = 64;
  struct Entry {
    MapKey key;
    CUtensorMap map;
  };
  static thread_local Entry table[kSlots];
  static thread_local int used = 0, next = 0;
  const MapKey key{base, n, d, rows, f16 ? 1 : 0, v.heads, v.batches, v.row, v.head, v.batch};
  for (int i = 0; i < used; ++i)
    if (table[i].key == key) {
      *m = table[i].map;
      return FHOB_OK;
    }
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_cuda_error_text("cuTensorMapEncodeTiled entry point not available");
    return FHOB_ERR_CUDA;
  }
  // strides of the three outer dims in bytes: multiples of 16, checked by the caller's validation
  // and once more by the driver
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(v.heads),
                        static_cast<cuuint64_t>(v.batches)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(v.row) * 2, static_cast<cuuint64_t>(v.head) * 2,
                           static_cast<cuuint64_t>(v.batch) * 2};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(m, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[96];
    snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    set_cuda_error_text(buf);
    return FHOB_ERR_CUDA;
  }
  Entry& e = table[next];
  e.key = key;
  e.map = *m;
  next = (next + 1) % kSlots;
  if (used < kSlots) ++used;
  return FHOB_OK;
}

// Raises the dynamic shared-memory limit of `kernel` once per device and host thread (it is a
// per-function, per-device attribute; setting it again on every launch costs a driver call).
template <class K>
int allow_smem(K kernel, int bytes) {
  constexpr int kSlots = 96;
  struct Entry {
    const void* fn;
    unsigned long long devices;
  };
  static thread_local Entry table[kSlots];
  static thread_local int used = 0;
  int dev = 0;
  FHOB_CUDA_OK(cudaGetDevice(&dev));
  const unsigned long long bit = (dev >= 0 && dev < 64) ? (1ull << dev) : 0;
  const void* fn = reinterpret_cast<const void*>(kernel);
  Entry* e = nullptr;
  for (int i = 0; i < used && !e; ++i)
    if (table[i].fn == fn) e = &table[i];
  if (e && bit && (e->devices & bit)) return FHOB_OK;
  FHOB_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  if (!e && used < kSlots) {
    e = &table[used++];
    e->fn = fn;
    e->devices = 0;
  }
  if (e) e->devices |= bit;
  return FHOB_OK;
}

}  // namespace
}  // namespace fhob
