// moba_route_static: the routing decision (selected chunks) with no workspace.
//
// Some hosts of this library cannot hand it device memory at call time: an
// inference server that froze its memory pool at start-up, a plugin that runs
// inside a stream-ordered region where the framework forbids allocation, or a
// small C client that only owns the input and output tensors.  For those
// callers the chunk means - the one intermediate the routing needs besides its
// inputs and outputs - live in a fixed array inside the library image instead
// of a caller-provided workspace.
//
// The array is part of the loaded module: every GPU that loads the library
// carries its 4 MiB until the process exits, whether this entry point is used
// or not.  All calls on a device share it and it keeps what the previous call
// wrote, so two calls whose kernels overlap on the GPU (different streams
// without an ordering between them) would race on it.  Nothing in it has to
// start at zero: the mean kernel writes every slot a call reads, zeros for
// slots that are not historical included.
#include <mutex>

#include "common.cuh"

namespace moba {
namespace {

constexpr size_t kStaticMeanElems = (size_t)2 << 20;     // 16-bit elements: slots * kv heads * head_dim <= 2 Mi (4 MiB)

static __device__ __align__(256) __nv_bfloat16 g_static_means[kStaticMeanElems];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
__nv_bfloat16* g_means_addr[kMaxDevices] = {nullptr};

// In host code `g_static_means` is only a handle for the symbol, not a device
// address.  The address on the current device is asked for once per device and
// remembered; the kernels receive that pointer.  cudaDeviceReset unloads the
// module and with it the array: a process that resets a device must not call
// this entry point on that device afterwards (the remembered address would be
// stale).
cudaError_t static_means_address(__nv_bfloat16** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_means_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_means);
    if (e != cudaSuccess) return e;
    g_means_addr[dev] = static_cast<__nv_bfloat16*>(ptr);
  }
  *out = g_means_addr[dev];
  return cudaSuccess;
}

}  // namespace
}  // namespace moba

extern "C" int moba_route_static(const moba_problem_t* p, const void* q, const void* k, const int32_t* cu_seqlens,
                                 int32_t* selected, void* stream) {
  using namespace moba;
  moba_dims_t dims;
  const int rc = moba_problem_dims(p, &dims);
  if (rc != MOBA_OK) return rc;
  if (!q || !k || !cu_seqlens || !selected) return MOBA_E_NULL;
  if (((uintptr_t)q | (uintptr_t)k) & 15) return MOBA_E_ALIGN;     // both are read with 16-byte loads
  if (dims.hist <= 0) return MOBA_OK;                      // nothing to select: `selected` has no rows
  if ((size_t)dims.slots * (size_t)p->num_kv_heads * (size_t)p->head_dim > kStaticMeanElems) return MOBA_E_STATIC_LIMIT;
  __nv_bfloat16* means = nullptr;
  cudaError_t e = static_means_address(&means);
  if (e != cudaSuccess) return (int)e;
  int st_rc = moba_chunk_means(p, k, cu_seqlens, means, stream);
  if (st_rc != MOBA_OK) return st_rc;
  return moba_gate_topk(p, q, means, cu_seqlens, selected, nullptr, stream);
}
