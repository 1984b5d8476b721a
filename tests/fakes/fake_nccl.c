/* A stand-in for libnccl used by the failure-detection test: every call succeeds and moves no data;
 * ncclCommGetAsyncError starts reporting ncclSystemError after FAKE_NCCL_FAIL_AFTER polls (never,
 * when the variable is unset); ncclCommAbort appends a line to the file FAKE_NCCL_LOG names.  The
 * failure is made on the host: no GPU work of this library exists that could hang or fault. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef int ncclResult_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef struct fake_comm { int rank, n, polls; } *ncclComm_t;

static void note(const char* what) {
  const char* path = getenv("FAKE_NCCL_LOG");
  if (!path) return;
  FILE* f = fopen(path, "a");
  if (!f) return;
  fprintf(f, "%s\n", what);
  fclose(f);
}

ncclResult_t ncclGetUniqueId(ncclUniqueId* id) { memset(id, 7, sizeof *id); return 0; }
ncclResult_t ncclCommInitRank(ncclComm_t* comm, int n, ncclUniqueId id, int rank) {
  (void)id;
  *comm = (ncclComm_t)calloc(1, sizeof **comm);
  (*comm)->rank = rank;
  (*comm)->n = n;
  note("init");
  return 0;
}
ncclResult_t ncclCommInitAll(ncclComm_t* comms, int n, const int* devs) {
  (void)devs;
  for (int i = 0; i < n; ++i) {
    comms[i] = (ncclComm_t)calloc(1, sizeof **comms);
    comms[i]->rank = i;
    comms[i]->n = n;
  }
  note("init_all");
  return 0;
}
ncclResult_t ncclGroupStart(void) { return 0; }
ncclResult_t ncclGroupEnd(void) { return 0; }
ncclResult_t ncclCommDestroy(ncclComm_t comm) { note("destroy"); free(comm); return 0; }
ncclResult_t ncclCommAbort(ncclComm_t comm) { note("abort"); free(comm); return 0; }
ncclResult_t ncclAllReduce(const void* s, void* r, size_t count, int dtype, int op, ncclComm_t comm, void* stream) {
  (void)s; (void)r; (void)count; (void)dtype; (void)op; (void)comm; (void)stream;
  note("allreduce");
  return 0;
}
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* async) {
  const char* after = getenv("FAKE_NCCL_FAIL_AFTER");
  comm->polls++;
  *async = (after && comm->polls > atoi(after)) ? 2 /* ncclSystemError */ : 0;
  return 0;
}
const char* ncclGetErrorString(ncclResult_t r) { return r == 2 ? "unhandled system error (fake)" : "fake nccl"; }
