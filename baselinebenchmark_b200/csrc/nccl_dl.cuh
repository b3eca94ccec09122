// NCCL entry points resolved at run time from the NCCL library that is already in the process
// (the host framework's) or, failing that, the system one: the context-parallel entry points
// then share the caller's communicator, and the library has no link-time dependency on NCCL.
// MOBA_NCCL_LIB names another library file (tests use a stand-in that records the calls).
#pragma once

#include <nccl.h>

namespace moba {

struct NcclApi {
  ncclResult_t (*GroupStart)();
  ncclResult_t (*GroupEnd)();
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*);
  ncclResult_t (*CommAbort)(ncclComm_t);
  const char* (*GetErrorString)(ncclResult_t);
};

// nullptr when no NCCL library could be loaded or a symbol is missing.
const NcclApi* nccl_api();

}  // namespace moba
