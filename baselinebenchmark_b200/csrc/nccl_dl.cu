// Run-time binding of the few NCCL functions the context-parallel path calls.
#include <dlfcn.h>

#include <cstdlib>
#include <mutex>

#include <cuda_runtime.h>

#include "nccl_dl.cuh"

namespace moba {

const NcclApi* nccl_api() {
  static NcclApi api;
  static bool ok = false;
  static std::once_flag once;
  std::call_once(once, []() {
    const char* names[3] = {std::getenv("MOBA_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (int i = 0; i < 3 && h == nullptr; ++i)
      if (names[i] != nullptr && names[i][0] != 0) h = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
    if (h == nullptr) return;
    bool all = true;
    auto get = [&](const char* sym) {
      void* f = dlsym(h, sym);
      if (f == nullptr) all = false;
      return f;
    };
    api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(get("ncclGroupStart"));
    api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(get("ncclGroupEnd"));
    api.Send = reinterpret_cast<decltype(api.Send)>(get("ncclSend"));
    api.Recv = reinterpret_cast<decltype(api.Recv)>(get("ncclRecv"));
    api.Broadcast = reinterpret_cast<decltype(api.Broadcast)>(get("ncclBroadcast"));
    api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(get("ncclCommGetAsyncError"));
    api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(get("ncclCommAbort"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(get("ncclGetErrorString"));
    ok = all;
  });
  return ok ? &api : nullptr;
}

}  // namespace moba
