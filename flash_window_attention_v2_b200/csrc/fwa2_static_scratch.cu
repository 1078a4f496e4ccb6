// Backward pass for callers that must not allocate device memory.
//
// Some hosts of this library cannot hand it a workspace: a plugin running inside a framework that
// owns the only allocator, a steady-state serving loop that forbids allocator traffic after
// warm-up, code in a context where cudaMalloc is not allowed.  For them the scratch the backward
// needs lives in a fixed array in the library's own device image: it exists on every GPU that
// loads the library, from load until exit, whether or not this entry point is ever used.
#include "../../include/fwa2.h"

#include <cuda_runtime.h>

#include <mutex>

namespace {

// 48 MiB: enough for windows of up to 256 tokens with 3 heads and a 64-window mask on a 148-SM
// part (147 partial dBias buffers of 256 KiB plus the transposed tables), the largest of the
// benchmark configurations.
__device__ __align__(256) static unsigned char g_fwa2_scratch[FWA2_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_scratch_ptr[kMaxDevices] = {};   // device address of the array, per device ordinal

}  // namespace

// In host code `g_fwa2_scratch` is only a handle for the runtime, not a device address; the
// address valid on the CURRENT device comes from cudaGetSymbolAddress, looked up once per device.
extern "C" int fwa2_backward_static_scratch(const fwa2_bwd_args* args, void* stream) {
  if (args == nullptr) return FWA2_ERR_NULL;
  if (args->struct_size != sizeof(fwa2_bwd_args) || args->abi_version != FWA2_ABI_VERSION) return FWA2_ERR_ABI;
  const size_t need = fwa2_bwd_workspace_bytes(args->bw, args->heads, args->n, args->n_windows,
                                               args->bias != nullptr, args->mask != nullptr);
  if (need == 0) return FWA2_ERR_SHAPE;
  if (need > static_cast<size_t>(FWA2_STATIC_SCRATCH_BYTES)) return FWA2_ERR_SCRATCH_LIMIT;

  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FWA2_ERR_LAUNCH;
  void* ptr = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
      void* p = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&p, g_fwa2_scratch);
      if (e != cudaSuccess || p == nullptr) return FWA2_ERR_LAUNCH;
      g_scratch_ptr[dev] = p;
    }
    ptr = g_scratch_ptr[dev];
  }

  // Every word of the scratch that the backward reads it has written earlier in the same call
  // (transposed tables, first-visit stores of the partial sums, one dLogitScale partial per
  // CTA), so nothing has to be cleared between calls even though the previous call's contents
  // are still there.
  fwa2_bwd_args local = *args;
  local.workspace = ptr;
  local.workspace_bytes = static_cast<size_t>(FWA2_STATIC_SCRATCH_BYTES);
  return fwa2_backward(&local, stream);
}
