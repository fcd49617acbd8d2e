/* A stand-in for libnccl used by the CPU tests of the communicator's failure handling.  It moves no data: every
 * entry point returns what the FAKE_NCCL_* environment variables script, and counts the calls so that a test can
 * check that a communicator was aborted.  Result codes follow NCCL's public enum (0 success, 1 unhandled CUDA
 * error, 3 internal error, 7 in progress). */
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

typedef struct { char internal[128]; } fake_id;
typedef struct { int polls; int aborted; } fake_comm;

static int g_aborts = 0, g_destroys = 0, g_inits = 0;
static fake_comm g_comm;

static int env_int(const char* name, int def) {
  const char* v = getenv(name);
  return v && v[0] ? atoi(v) : def;
}

int ncclGetUniqueId(fake_id* id) { memset(id, 0x5A, sizeof(*id)); return 0; }
int ncclCommInitRank(void** comm, int nranks, fake_id id, int rank) {
  (void)nranks; (void)id; (void)rank;
  g_inits++; g_comm.polls = 0; g_comm.aborted = 0; *comm = &g_comm;
  return env_int("FAKE_NCCL_INIT_RESULT", 0);
}
int ncclCommInitRankConfig(void** comm, int nranks, fake_id id, int rank, void* config) {
  /* the record must carry NCCL's magic and ask for non-blocking operation */
  const unsigned* words = (const unsigned*)((const char*)config + sizeof(size_t));
  const int blocking = *(const int*)((const char*)config + sizeof(size_t) + 8);
  if (words[0] != 0xcafebeefu || blocking != 0 || env_int("FAKE_NCCL_REFUSE_CONFIG", 0)) return 4;
  (void)nranks; (void)id; (void)rank;
  g_inits++; g_comm.polls = 0; g_comm.aborted = 0; *comm = &g_comm;
  return env_int("FAKE_NCCL_INIT_RESULT", 7);       /* in progress, like the real library */
}
/* in progress for FAKE_NCCL_POLLS polls (-1: for ever), then FAKE_NCCL_ASYNC_RESULT */
int ncclCommGetAsyncError(void* comm, int* state) {
  fake_comm* c = (fake_comm*)comm;
  const int polls = env_int("FAKE_NCCL_POLLS", 3);
  c->polls++;
  *state = (polls < 0 || c->polls <= polls) ? 7 : env_int("FAKE_NCCL_ASYNC_RESULT", 0);
  return 0;
}
int ncclCommAbort(void* comm) { ((fake_comm*)comm)->aborted = 1; g_aborts++; return 0; }
int ncclCommDestroy(void* comm) { (void)comm; g_destroys++; return 0; }
int ncclAllGather(const void* s, void* r, size_t n, int dt, void* comm, void* stream) {
  (void)s; (void)r; (void)n; (void)dt; (void)stream;
  ((fake_comm*)comm)->polls = 0;
  return env_int("FAKE_NCCL_ENQUEUE_RESULT", 7);
}
int ncclAllReduce(const void* s, void* r, size_t n, int dt, int op, void* comm, void* stream) {
  (void)s; (void)r; (void)n; (void)dt; (void)op; (void)stream;
  ((fake_comm*)comm)->polls = 0;
  return env_int("FAKE_NCCL_ENQUEUE_RESULT", 7);
}
const char* ncclGetErrorString(int r) { return r == 7 ? "in progress" : r == 3 ? "internal error (fake)" : "error (fake)"; }

int fake_nccl_aborts(void) { return g_aborts; }
int fake_nccl_destroys(void) { return g_destroys; }
int fake_nccl_inits(void) { return g_inits; }
