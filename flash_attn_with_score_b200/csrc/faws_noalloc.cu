// faws_attention_with_col_sum_noalloc: the column-sum operator for callers that cannot
// provide scratch memory.
//
// Who needs it: a host application that has handed the whole device to its own pool
// allocator and forbids plugins from calling cudaMalloc; a serving loop that cannot take
// the device-wide synchronisation a cudaMalloc / cudaFree implies; a C plugin interface
// that passes the tensors' pointers and nothing else, so there is no allocator to ask for
// the workspace that faws_attention_with_col_sum wants.  For them the per-query-tile
// partial sums live in a fixed array inside the library image instead.
//
// Cost and limits: the array is FAWS_NOALLOC_SCRATCH_BYTES (8 MiB) of device memory on every
// GPU that loads the library, held until the process exits.  Problems whose partial sums do
// not fit are refused with FAWS_ETOOLARGE.  All calls on a device share the one array, so
// two calls whose kernels can overlap on the GPU (different streams, no ordering between
// them) race on it; serialise them.  The array keeps the previous call's contents; no part
// of it has to be zero on entry because every call writes each partial before the reduce
// kernel of the same call reads it.
//
// The first call on each device looks the array's device address up
// (cudaGetSymbolAddress) and caches it; make that first call before any stream capture.
// Nothing here, nor in the entry point it forwards to, calls cudaMalloc, cudaFree or an
// allocating library routine.
#include <cuda_runtime.h>

#include <mutex>

#include "faws.h"

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device
// pointer and must never be passed to a kernel directly.
static __device__ __align__(256) unsigned char g_noalloc_scratch[FAWS_NOALLOC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;

// Device address of g_noalloc_scratch on the current device (set-up once per device).
void* scratch_of_current_device() {
  static void* addr[kMaxDevices] = {nullptr};
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess) return nullptr;
    addr[dev] = ptr;
  }
  return addr[dev];
}

}  // namespace

extern "C" int faws_attention_with_col_sum_noalloc(const faws_problem* p, float* col_sum,
                                                   int32_t per_q_head, void* stream) {
  if (p == nullptr || col_sum == nullptr) return FAWS_EINVAL;
  // 0 for an invalid problem; the forwarded call then reports the precise error.
  const size_t need = faws_workspace_bytes(FAWS_OP_COL_SUM, p, 0);
  if (need > (size_t)FAWS_NOALLOC_SCRATCH_BYTES) return FAWS_ETOOLARGE;
  void* scratch = scratch_of_current_device();
  if (scratch == nullptr) return FAWS_ECUDA;
  return faws_attention_with_col_sum(p, col_sum, per_q_head, scratch, (size_t)FAWS_NOALLOC_SCRATCH_BYTES,
                                     stream);
}
