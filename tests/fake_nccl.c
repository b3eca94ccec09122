/* Stand-in for libnccl used by tests/test_cp_abi.py on a machine without GPUs: it has the
 * entry points the library binds at run time and records what was called.
 * FAKE_NCCL_ASYNC_ERROR sets the state ncclCommGetAsyncError reports; ncclCommAbort appends a
 * line to the file FAKE_NCCL_LOG names. */
#include <stdio.h>
#include <stdlib.h>

typedef int ncclResult_t;
typedef void* ncclComm_t;

static void note(const char* what) {
  const char* path = getenv("FAKE_NCCL_LOG");
  if (!path) return;
  FILE* f = fopen(path, "a");
  if (f) { fprintf(f, "%s\n", what); fclose(f); }
}

ncclResult_t ncclGroupStart(void) { return 0; }
ncclResult_t ncclGroupEnd(void) { return 0; }
ncclResult_t ncclSend(const void* b, size_t n, int t, int peer, ncclComm_t c, void* s) { note("send"); return 0; }
ncclResult_t ncclRecv(void* b, size_t n, int t, int peer, ncclComm_t c, void* s) { note("recv"); return 0; }
ncclResult_t ncclBroadcast(const void* a, void* b, size_t n, int t, int root, ncclComm_t c, void* s) { note("broadcast"); return 0; }
ncclResult_t ncclCommGetAsyncError(ncclComm_t c, ncclResult_t* state) {
  const char* e = getenv("FAKE_NCCL_ASYNC_ERROR");
  *state = e ? atoi(e) : 0;
  return 0;
}
ncclResult_t ncclCommAbort(ncclComm_t c) { note("abort"); return 0; }
const char* ncclGetErrorString(ncclResult_t r) { return "fake"; }
