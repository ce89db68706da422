// tpa_fwd_static_scratch: the staged tensor-core forward for callers that cannot hand over a
// scratch buffer they allocated.
//
// Who that is.  The intended binding of this library is an XLA custom call (jax.ffi).  Inside
// such a handler the device memory belongs to XLA's allocator, which by default has already
// reserved most of the GPU, so a cudaMalloc made from the handler can fail or fragment that
// pool, and the handler only sees the operand and result buffers XLA chose to give it.  The
// same holds for any embedder that runs with a fixed device-memory budget.  Those callers
// cannot size and pass the workspace that tpa_fwd wants for its staged Q/K/V tiles.
//
// What this file does about it.  The scratch lives in the library image itself: one
// file-scope __device__ array of TPA_STATIC_SCRATCH_BYTES.  Every GPU whose context loads the
// library holds that much memory until the process exits, which is why the size is modest and
// problems that need more are refused.  No cudaMalloc, cudaFree or other allocating routine is
// called here or below (tpa_fwd only sets a function attribute, enqueues one memset of the
// 256-byte status block and launches two kernels).
//
// In host code the array's name is a host-side handle, not a device address, so the address
// the kernels get comes from cudaGetSymbolAddress, looked up once per device under a mutex by
// the first call made with that device current.  That first call does this one-time lookup;
// make it during start-up, before any stream capture is begun.
//
// All calls on a device share the one array and it keeps whatever the previous call left.
// The only part that must start at zero, the status block at its head, is cleared on the
// stream by every call; the staged tiles are fully rewritten for the shape at hand before they
// are read.  Two calls that overlap on the same GPU (different streams, or different threads)
// would stage into the same bytes and race: serialise them.
#include <mutex>

#include "tpa_common.cuh"

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[TPA_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_scratch_addr[kMaxDevices] = {};

// Device address of the array on the current device; nullptr (and *err set) on failure.
void* scratch_for_current_device(cudaError_t* err) {
  int dev = -1;
  *err = cudaGetDevice(&dev);
  if (*err != cudaSuccess) return nullptr;
  if (dev < 0 || dev >= kMaxDevices) {
    *err = cudaErrorInvalidDevice;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    *err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (*err != cudaSuccess) return nullptr;
    g_scratch_addr[dev] = ptr;
  }
  return g_scratch_addr[dev];
}

}  // namespace

extern "C" int tpa_fwd_static_scratch(const TpaFwdArgs* args, void* stream) {
  if (args == nullptr || args->struct_size != sizeof(TpaFwdArgs)) return TPA_ERR_BAD_ARG;
  TpaFwdArgs a = *args;
  a.kernel = TPA_KERNEL_SM100_STAGED;  // the variant whose scratch this entry point supplies
  TpaKernelInfo info;
  const int st = tpa_query_kernel(&a, &info);  // same validation and shape rules as tpa_fwd
  if (st != TPA_OK) return st;
  if (tpa_fwd_workspace_bytes(&a) > (size_t)TPA_STATIC_SCRATCH_BYTES) return TPA_ERR_STATIC_SCRATCH;
  cudaError_t err = cudaSuccess;
  void* scratch = scratch_for_current_device(&err);
  // the first look-up on a device is where the array is instantiated, the step most likely to
  // fail in a process whose memory is already reserved: its error text must not be lost
  if (scratch == nullptr) return tpa::fail_cuda(err);
  return tpa_fwd(&a, scratch, (size_t)TPA_STATIC_SCRATCH_BYTES, stream);
}

// The status block of tpa_fwd_static_scratch sits at the head of the static array, whose address
// no caller has; this reads it for the current device (same contract as tpa_read_status).
extern "C" int tpa_read_status_static_scratch(void* stream, uint32_t detail[4]) {
  cudaError_t err = cudaSuccess;
  void* scratch = scratch_for_current_device(&err);
  if (scratch == nullptr) return tpa::fail_cuda(err);
  return tpa_read_status(scratch, stream, detail);
}
