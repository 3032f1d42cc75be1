/* Stand-in for libnccl used by the CPU tests of the native process group: one rank, collectives are host copies,
   the asynchronous error state and the result of the next call can be set from the test. */
#include <stdlib.h>
#include <string.h>
static int g_async_error = 0, g_next_rc = 0, g_aborts = 0, g_calls = 0;
typedef struct { char internal[128]; } uid_t128;
static size_t esize(int dt) { static const size_t s[] = {1, 1, 4, 4, 8, 8, 2, 4, 8, 2}; return dt >= 0 && dt < 10 ? s[dt] : 4; }
void fake_nccl_set(int async_error, int next_rc) { g_async_error = async_error; g_next_rc = next_rc; }
int fake_nccl_aborts(void) { return g_aborts; }
int fake_nccl_calls(void) { return g_calls; }
int ncclGetUniqueId(uid_t128* id) { memset(id, 7, sizeof(*id)); return 0; }
int ncclCommInitRank(void** comm, int n, uid_t128 id, int rank) { (void)id; if (n != 1 || rank != 0) return 5; *comm = malloc(8); return 0; }
int ncclCommDestroy(void* c) { free(c); return 0; }
int ncclCommAbort(void* c) { ++g_aborts; free(c); return 0; }
int ncclCommGetAsyncError(void* c, int* e) { (void)c; *e = g_async_error; return 0; }
static int copy(const void* s, void* r, size_t n, int dt) { ++g_calls; if (g_next_rc) { int rc = g_next_rc; g_next_rc = 0; return rc; } if (s && r && s != r) memcpy(r, s, n * esize(dt)); return 0; }
int ncclAllReduce(const void* s, void* r, size_t n, int dt, int op, void* c, void* st) { (void)op; (void)c; (void)st; return copy(s, r, n, dt); }
int ncclAllGather(const void* s, void* r, size_t n, int dt, void* c, void* st) { (void)c; (void)st; return copy(s, r, n, dt); }
int ncclReduceScatter(const void* s, void* r, size_t n, int dt, int op, void* c, void* st) { (void)op; (void)c; (void)st; return copy(s, r, n, dt); }
int ncclBroadcast(const void* s, void* r, size_t n, int dt, int root, void* c, void* st) { (void)root; (void)c; (void)st; return copy(s, r, n, dt); }
int ncclReduce(const void* s, void* r, size_t n, int dt, int op, int root, void* c, void* st) { (void)op; (void)root; (void)c; (void)st; return copy(s, r, n, dt); }
int ncclSend(const void* s, size_t n, int dt, int p, void* c, void* st) { (void)s; (void)n; (void)dt; (void)p; (void)c; (void)st; ++g_calls; return 0; }
int ncclRecv(void* r, size_t n, int dt, int p, void* c, void* st) { (void)r; (void)n; (void)dt; (void)p; (void)c; (void)st; ++g_calls; return 0; }
int ncclGroupStart(void) { return 0; }
int ncclGroupEnd(void) { return 0; }
