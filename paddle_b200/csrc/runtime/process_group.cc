// Native process group over NCCL: communicator bring-up, collectives and point-to-point calls issued on a dedicated
// communication stream (or on the caller's compute stream), Task objects whose completion is a CUDA event, bounded
// host-side waits that also watch the communicator's asynchronous error state, and abort.
//
// Counterpart of ProcessGroupNCCL (paddle/fluid/distributed/collective/process_group_nccl.cc: Collective :899-993,
// Point2Point :996, task Wait / Synchronize :100-140) and NCCLCommContext
// (paddle/phi/core/distributed/nccl_comm_context.cc:91-249).  Stream semantics of the reference:
//   use_calc_stream = true : the call is enqueued on the caller's stream, nothing to wait for
//   use_calc_stream = false: the comm stream first waits for what the compute stream has enqueued so far (event),
//                            runs the call, records a completion event; Task::Wait makes the compute stream wait
//                            for that event (device-side) or blocks the host until it has fired (bounded)
// NCCL and the CUDA runtime are reached through dlopen / dlsym (the reference's dynload layer,
// paddle/phi/backends/dynload/nccl.h): the library has no link-time dependency on either, and the tests substitute
// small stand-ins for both to drive the timeout / error / abort paths on a machine without GPUs.
#include <dlfcn.h>
#include <stdint.h>
#include <string.h>

#include <chrono>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#define PD_EXPORT extern "C" __attribute__((visibility("default")))

extern "C" {
int64_t pd_watchdog_task_create(int group, const char* name, int64_t bytes);
void pd_watchdog_task_started(int64_t id);
void pd_watchdog_task_finished(int64_t id);
}

namespace {

struct UniqueId { char internal[128]; };          // same layout as ncclUniqueId
typedef void* Comm;
typedef void* Stream;
typedef void* Event;

// ---- function tables filled by dlsym
struct NcclApi {
  int (*GetUniqueId)(UniqueId*);
  int (*CommInitRank)(Comm*, int, UniqueId, int);
  int (*CommDestroy)(Comm);
  int (*CommAbort)(Comm);
  int (*CommGetAsyncError)(Comm, int*);
  int (*AllReduce)(const void*, void*, size_t, int, int, Comm, Stream);
  int (*AllGather)(const void*, void*, size_t, int, Comm, Stream);
  int (*ReduceScatter)(const void*, void*, size_t, int, int, Comm, Stream);
  int (*Broadcast)(const void*, void*, size_t, int, int, Comm, Stream);
  int (*Reduce)(const void*, void*, size_t, int, int, int, Comm, Stream);
  int (*Send)(const void*, size_t, int, int, Comm, Stream);
  int (*Recv)(void*, size_t, int, int, Comm, Stream);
  int (*GroupStart)();
  int (*GroupEnd)();
  bool ok = false;
} g_nccl;

struct CudaApi {
  int (*SetDevice)(int);
  int (*StreamCreateWithFlags)(Stream*, unsigned);
  int (*StreamDestroy)(Stream);
  int (*EventCreateWithFlags)(Event*, unsigned);
  int (*EventDestroy)(Event);
  int (*EventRecord)(Event, Stream);
  int (*EventQuery)(Event);
  int (*StreamWaitEvent)(Stream, Event, unsigned);
  bool ok = false;
} g_cuda;

template <typename F>
bool sym(void* lib, const char* name, F* out) {
  *out = reinterpret_cast<F>(dlsym(lib, name));
  return *out != nullptr;
}

struct Task {
  int64_t id = 0;
  Event done = nullptr;           // null for calls on the compute stream
  int64_t wd_id = 0;
  bool finished = false;
};

struct ProcessGroup {
  Comm comm = nullptr;
  Stream comm_stream = nullptr;
  int rank = 0, nranks = 1, device = 0;
  bool aborted = false;
  int64_t next_task = 1;
  std::map<int64_t, Task> tasks;
  std::mutex mu;
};

constexpr unsigned kStreamNonBlocking = 1, kEventDisableTiming = 2;

}  // namespace

// Load the two libraries.  Paths may be null: the usual sonames are tried (an already loaded copy is reused).
PD_EXPORT int pd_pg_load(const char* nccl_path, const char* cudart_path) {
  const char* nccl_names[] = {nccl_path, "libnccl.so.2", "libnccl.so"};
  void* nl = nullptr;
  for (const char* n : nccl_names)
    if (n != nullptr && (nl = dlopen(n, RTLD_NOW | RTLD_GLOBAL)) != nullptr) break;
  const char* rt_names[] = {cudart_path, "libcudart.so.12", "libcudart.so.13", "libcudart.so"};
  void* cl = nullptr;
  for (const char* n : rt_names)
    if (n != nullptr && (cl = dlopen(n, RTLD_NOW | RTLD_GLOBAL)) != nullptr) break;
  if (nl == nullptr) return -1;
  if (cl == nullptr) return -2;
  NcclApi& a = g_nccl;
  a.ok = sym(nl, "ncclGetUniqueId", &a.GetUniqueId) && sym(nl, "ncclCommInitRank", &a.CommInitRank) &&
         sym(nl, "ncclCommDestroy", &a.CommDestroy) && sym(nl, "ncclCommAbort", &a.CommAbort) &&
         sym(nl, "ncclCommGetAsyncError", &a.CommGetAsyncError) && sym(nl, "ncclAllReduce", &a.AllReduce) &&
         sym(nl, "ncclAllGather", &a.AllGather) && sym(nl, "ncclReduceScatter", &a.ReduceScatter) &&
         sym(nl, "ncclBroadcast", &a.Broadcast) && sym(nl, "ncclReduce", &a.Reduce) && sym(nl, "ncclSend", &a.Send) &&
         sym(nl, "ncclRecv", &a.Recv) && sym(nl, "ncclGroupStart", &a.GroupStart) && sym(nl, "ncclGroupEnd", &a.GroupEnd);
  CudaApi& c = g_cuda;
  c.ok = sym(cl, "cudaSetDevice", &c.SetDevice) && sym(cl, "cudaStreamCreateWithFlags", &c.StreamCreateWithFlags) &&
         sym(cl, "cudaStreamDestroy", &c.StreamDestroy) && sym(cl, "cudaEventCreateWithFlags", &c.EventCreateWithFlags) &&
         sym(cl, "cudaEventDestroy", &c.EventDestroy) && sym(cl, "cudaEventRecord", &c.EventRecord) &&
         sym(cl, "cudaEventQuery", &c.EventQuery) && sym(cl, "cudaStreamWaitEvent", &c.StreamWaitEvent);
  if (!a.ok) return -3;
  if (!c.ok) return -4;
  return 0;
}

PD_EXPORT int pd_pg_unique_id(char* out128) {
  if (!g_nccl.ok) return -1;
  UniqueId id;
  memset(&id, 0, sizeof(id));
  if (g_nccl.GetUniqueId(&id) != 0) return -2;
  memcpy(out128, id.internal, 128);
  return 0;
}

PD_EXPORT void* pd_pg_create(const char* id128, int rank, int nranks, int device) {
  if (!g_nccl.ok || !g_cuda.ok) return nullptr;
  if (g_cuda.SetDevice(device) != 0) return nullptr;
  auto* pg = new ProcessGroup();
  pg->rank = rank;
  pg->nranks = nranks;
  pg->device = device;
  UniqueId id;
  memcpy(id.internal, id128, 128);
  if (g_nccl.CommInitRank(&pg->comm, nranks, id, rank) != 0 ||
      g_cuda.StreamCreateWithFlags(&pg->comm_stream, kStreamNonBlocking) != 0) {
    delete pg;
    return nullptr;
  }
  return pg;
}

// kind: 0 all_reduce, 1 all_gather (count = elements per rank), 2 reduce_scatter (count = elements per rank),
//       3 broadcast (root), 4 reduce (root), 5 send (peer), 6 recv (peer)
// dtype / op: NCCL's enum values (ncclDataType_t / ncclRedOp_t).  Returns a task id > 0, or a negative error:
//   -1 bad handle / aborted, -2 CUDA error, -3 NCCL error (the NCCL result is stored in *nccl_rc when given).
PD_EXPORT int64_t pd_pg_collective(void* h, int kind, const void* send, void* recv, int64_t count, int dtype, int op,
                                   int root_or_peer, void* calc_stream, int use_calc_stream, int* nccl_rc) {
  auto* pg = static_cast<ProcessGroup*>(h);
  if (pg == nullptr || pg->aborted) return -1;
  Stream st = use_calc_stream ? calc_stream : pg->comm_stream;
  Event done = nullptr;
  if (!use_calc_stream) {
    // comm stream waits for everything the compute stream has enqueued so far (the operands)
    Event ready = nullptr;
    if (g_cuda.EventCreateWithFlags(&ready, kEventDisableTiming) != 0) return -2;
    if (g_cuda.EventRecord(ready, calc_stream) != 0 || g_cuda.StreamWaitEvent(pg->comm_stream, ready, 0) != 0) {
      g_cuda.EventDestroy(ready);
      return -2;
    }
    g_cuda.EventDestroy(ready);      // destruction is deferred by the runtime until the event has completed
  }
  static const char* names[] = {"all_reduce", "all_gather", "reduce_scatter", "broadcast", "reduce", "send", "recv"};
  const int64_t wd = pd_watchdog_task_create(0, kind >= 0 && kind < 7 ? names[kind] : "?", count);
  int rc = 0;
  const size_t n = static_cast<size_t>(count);
  switch (kind) {
    case 0: rc = g_nccl.AllReduce(send, recv, n, dtype, op, pg->comm, st); break;
    case 1: rc = g_nccl.AllGather(send, recv, n, dtype, pg->comm, st); break;
    case 2: rc = g_nccl.ReduceScatter(send, recv, n, dtype, op, pg->comm, st); break;
    case 3: rc = g_nccl.Broadcast(send, recv, n, dtype, root_or_peer, pg->comm, st); break;
    case 4: rc = g_nccl.Reduce(send, recv, n, dtype, op, root_or_peer, pg->comm, st); break;
    case 5: rc = g_nccl.Send(send, n, dtype, root_or_peer, pg->comm, st); break;
    case 6: rc = g_nccl.Recv(recv, n, dtype, root_or_peer, pg->comm, st); break;
    default: rc = -1;
  }
  if (nccl_rc != nullptr) *nccl_rc = rc;
  if (rc != 0) {
    pd_watchdog_task_finished(wd);
    return -3;
  }
  pd_watchdog_task_started(wd);
  if (!use_calc_stream) {
    if (g_cuda.EventCreateWithFlags(&done, kEventDisableTiming) != 0 || g_cuda.EventRecord(done, pg->comm_stream) != 0)
      return -2;
  }
  std::lock_guard<std::mutex> g(pg->mu);
  Task t;
  t.id = pg->next_task++;
  t.done = done;
  t.wd_id = wd;
  t.finished = use_calc_stream != 0;
  if (t.finished) pd_watchdog_task_finished(wd);
  pg->tasks[t.id] = t;
  return t.id;
}

PD_EXPORT int pd_pg_group_start() { return g_nccl.ok ? g_nccl.GroupStart() : -1; }
PD_EXPORT int pd_pg_group_end() { return g_nccl.ok ? g_nccl.GroupEnd() : -1; }

// 1 = the communicator reports an asynchronous error (a peer died, a network fault), 0 = healthy, -1 bad handle
PD_EXPORT int pd_pg_async_error(void* h) {
  auto* pg = static_cast<ProcessGroup*>(h);
  if (pg == nullptr || pg->comm == nullptr) return -1;
  int e = 0;
  if (g_nccl.CommGetAsyncError(pg->comm, &e) != 0) return 1;
  return e != 0 ? 1 : 0;
}

// timeout_ms < 0 : device-side wait only - the compute stream waits for the task, the host returns at once
// timeout_ms >= 0: the host polls until the task's event has fired.  Returns 0 done, 1 timeout, 2 communicator error,
//                  -1 unknown task, -2 CUDA error.  A finished task is forgotten.
PD_EXPORT int pd_pg_task_wait(void* h, int64_t task, int timeout_ms, void* calc_stream) {
  auto* pg = static_cast<ProcessGroup*>(h);
  if (pg == nullptr) return -1;
  Task t;
  {
    std::lock_guard<std::mutex> g(pg->mu);
    auto it = pg->tasks.find(task);
    if (it == pg->tasks.end()) return -1;
    t = it->second;
  }
  auto forget = [&]() {
    std::lock_guard<std::mutex> g(pg->mu);
    pg->tasks.erase(task);
    if (t.done != nullptr) g_cuda.EventDestroy(t.done);
    if (!t.finished) pd_watchdog_task_finished(t.wd_id);
  };
  if (t.done == nullptr) {
    forget();
    return 0;
  }
  if (timeout_ms < 0) {
    if (g_cuda.StreamWaitEvent(calc_stream, t.done, 0) != 0) return -2;
    forget();      // the event's resources are released by the runtime once the wait has been satisfied
    return 0;
  }
  const auto t0 = std::chrono::steady_clock::now();
  while (true) {
    const int q = g_cuda.EventQuery(t.done);
    if (q == 0) {
      forget();
      return 0;
    }
    if (q != 600 /* cudaErrorNotReady */) return -2;
    if (pd_pg_async_error(pg) == 1) return 2;
    const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
    if (ms > timeout_ms) return 1;
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

PD_EXPORT int pd_pg_task_done(void* h, int64_t task) {
  auto* pg = static_cast<ProcessGroup*>(h);
  if (pg == nullptr) return -1;
  std::lock_guard<std::mutex> g(pg->mu);
  auto it = pg->tasks.find(task);
  if (it == pg->tasks.end()) return 1;
  if (it->second.done == nullptr) return 1;
  return g_cuda.EventQuery(it->second.done) == 0 ? 1 : 0;
}

// Tear the communicator down without waiting for outstanding calls (after a timeout or a peer's error report):
// kernels of this communicator that are still waiting for a peer end, every later call on the group is refused.
PD_EXPORT int pd_pg_abort(void* h) {
  auto* pg = static_cast<ProcessGroup*>(h);
  if (pg == nullptr) return -1;
  if (pg->aborted) return 0;
  pg->aborted = true;
  const int rc = pg->comm != nullptr ? g_nccl.CommAbort(pg->comm) : 0;
  pg->comm = nullptr;
  std::lock_guard<std::mutex> g(pg->mu);
  for (auto& kv : pg->tasks)
    if (!kv.second.finished) pd_watchdog_task_finished(kv.second.wd_id);
  return rc;
}

PD_EXPORT int pd_pg_inflight(void* h) {
  auto* pg = static_cast<ProcessGroup*>(h);
  if (pg == nullptr) return -1;
  std::lock_guard<std::mutex> g(pg->mu);
  return static_cast<int>(pg->tasks.size());
}

PD_EXPORT void pd_pg_destroy(void* h) {
  auto* pg = static_cast<ProcessGroup*>(h);
  if (pg == nullptr) return;
  if (pg->comm != nullptr && !pg->aborted) g_nccl.CommDestroy(pg->comm);
  if (pg->comm_stream != nullptr) g_cuda.StreamDestroy(pg->comm_stream);
  for (auto& kv : pg->tasks)
    if (kv.second.done != nullptr) g_cuda.EventDestroy(kv.second.done);
  delete pg;
}
