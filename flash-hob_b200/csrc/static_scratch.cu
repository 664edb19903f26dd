// fhob_bwdbwd_static_scratch: the whole operator for callers that cannot allocate.
//
// Some hosts of this library own every byte of device memory themselves and
// forbid cudaMalloc from inside an operator call: runtimes that hand out
// memory from one pre-sized arena, plug-ins called from inside another
// framework's allocator-managed region, and real-time style loops where an
// allocation (which may synchronise the device) is not acceptable.  Such a
// caller can already pass its own workspace to fhob_bwdbwd; this entry point
// serves the ones that have nowhere to take even that from.  The row-vector
// scratch of the operator lives in a fixed array inside the library image
// instead, so the call needs nothing but the caller's inputs and outputs.
#include <mutex>

#include "fhob_common.cuh"

namespace {

// Status header + four fp32 row vectors of FHOB_STATIC_SCRATCH_MAX_ROWS entries + the tail pad
// the key-tiled pass may read past the last head.  About 4 MiB, resident on every GPU that loads
// the library, for the life of the process.
constexpr size_t kScratchBytes = fhob::kWorkspaceHeaderBytes +
                                 4 * sizeof(float) * static_cast<size_t>(FHOB_STATIC_SCRATCH_MAX_ROWS) +
                                 fhob::kWorkspaceTailBytes;

static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {};  // device address of g_static_scratch, per device ordinal

// In host code `g_static_scratch` is only a handle for the runtime, not a device address, so the
// address each device gave the array is looked up once, with that device current.
int scratch_for_current_device(void** out) {
  int dev = -1;
  FHOB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return FHOB_ERR_ARG;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    FHOB_CUDA_OK(cudaGetSymbolAddress(&ptr, g_static_scratch));
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return FHOB_OK;
}

}  // namespace

extern "C" int fhob_bwdbwd_static_scratch(const FhobProblem* p, void* stream) {
  if (!p) return FHOB_ERR_ARG;
  if (p->bh <= 0 || p->n_q <= 0) return FHOB_ERR_ARG;
  const long long rows = static_cast<long long>(p->bh) * static_cast<long long>(fhob::row_stride(p->n_q));
  if (rows > FHOB_STATIC_SCRATCH_MAX_ROWS) return FHOB_ERR_STATIC_LIMIT;
  void* scratch = nullptr;
  int st = scratch_for_current_device(&scratch);
  if (st != FHOB_OK) return st;
  FhobProblem q = *p;  // the caller's workspace fields are ignored
  q.workspace = scratch;
  q.workspace_bytes = kScratchBytes;
  // Nothing in the array has to be pre-cleared by hand: the pre-pass zeroes the status word and
  // every row vector entry a pass reads was written earlier in the same call.
  return fhob_bwdbwd(&q, stream);
}


// The device status word of the built-in array (its first four bytes), for the current device.
// Synchronises `stream`; allocates nothing.
extern "C" int fhob_static_scratch_status(void* stream) {
  void* scratch = nullptr;
  int st = scratch_for_current_device(&scratch);
  if (st != FHOB_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int host = 0;
  FHOB_CUDA_OK(cudaMemcpyAsync(&host, scratch, sizeof(int), cudaMemcpyDeviceToHost, s));
  FHOB_CUDA_OK(cudaStreamSynchronize(s));
  return host;
}
