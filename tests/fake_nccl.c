/* A stand-in for libnccl used ONLY by the host-side tests of the communicator's deadline and abort logic
 * (tests/test_comm_deadline.py points GB_NCCL_LIBRARY at the library built from this file).  It moves no data and
 * touches no GPU: each call appends its name to the file named by FAKE_NCCL_LOG and answers what FAKE_NCCL_MODE asks:
 *   ok              every call succeeds at once
 *   hang_init       ncclCommInitRankConfig answers "in progress" and the communicator never becomes ready
 *   hang_allreduce  ncclAllReduce answers "in progress" and never settles (a peer that never joined)
 *   error           the communicator reports an asynchronous system error after ncclAllReduce
 * Result codes and enum values are those of nccl.h (ncclSuccess 0, ncclSystemError 2, ncclInProgress 7). */
#include <stddef.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct { char internal[128]; } ncclUniqueId;
typedef void* ncclComm_t;

static int pending = 0;   /* 1: the last call is still "in progress" */
static int failed = 0;

static const char* mode(void) {
  const char* m = getenv("FAKE_NCCL_MODE");
  return m ? m : "ok";
}
static void note(const char* what) {
  const char* path = getenv("FAKE_NCCL_LOG");
  if (!path) return;
  FILE* f = fopen(path, "a");
  if (!f) return;
  fprintf(f, "%s\n", what);
  fclose(f);
}

int ncclGetUniqueId(ncclUniqueId* id) {
  note("ncclGetUniqueId");
  memset(id, 0x5a, sizeof(*id));
  return 0;
}
int ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank, void* config) {
  (void)nranks; (void)id; (void)rank; (void)config;
  note("ncclCommInitRankConfig");
  *comm = (ncclComm_t)&pending;
  if (strcmp(mode(), "hang_init") == 0) { pending = 1; return 7; }
  return 0;
}
int ncclCommGetAsyncError(ncclComm_t comm, int* state) {
  (void)comm;
  *state = failed ? 2 : (pending ? 7 : 0);
  return 0;
}
int ncclAllReduce(const void* src, void* dst, size_t count, int dtype, int op, ncclComm_t comm, void* stream) {
  (void)src; (void)dst; (void)comm; (void)stream;
  char line[96];
  snprintf(line, sizeof(line), "ncclAllReduce count=%zu dtype=%d op=%d", count, dtype, op);
  note(line);
  if (strcmp(mode(), "hang_allreduce") == 0) { pending = 1; return 7; }
  if (strcmp(mode(), "error") == 0) { failed = 1; return 7; }
  return 0;
}
int ncclCommAbort(ncclComm_t comm) { (void)comm; note("ncclCommAbort"); pending = 0; return 0; }
int ncclCommDestroy(ncclComm_t comm) { (void)comm; note("ncclCommDestroy"); return 0; }
