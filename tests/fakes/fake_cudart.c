/* Stand-in for libcudart used by the CPU tests of the native process group: streams and events are counters; while
   "stalled" is set, events recorded on a non-null stream never complete (a collective that waits for a peer). */
#include <stdlib.h>
static int g_stalled = 0;
typedef struct { int ready; } ev_t;
void fake_cuda_stall(int on) { g_stalled = on; }
int cudaSetDevice(int d) { (void)d; return 0; }
int cudaStreamCreateWithFlags(void** s, unsigned f) { (void)f; *s = malloc(8); return 0; }
int cudaStreamDestroy(void* s) { free(s); return 0; }
int cudaEventCreateWithFlags(void** e, unsigned f) { (void)f; ev_t* v = malloc(sizeof(ev_t)); v->ready = 1; *e = v; return 0; }
int cudaEventDestroy(void* e) { free(e); return 0; }
int cudaEventRecord(void* e, void* s) { ((ev_t*)e)->ready = (s == 0 || !g_stalled) ? 1 : 0; return 0; }
int cudaEventQuery(void* e) { ev_t* v = e; if (!v->ready && !g_stalled) v->ready = 1; return v->ready ? 0 : 600; }
int cudaStreamWaitEvent(void* s, void* e, unsigned f) { (void)s; (void)e; (void)f; return 0; }
