// Host runtime pieces with a C ABI:
//   * flag registry initialised from FLAGS_<name> environment variables (paddle/common/flags.cc)
//   * gradient bucket assignment for the data-parallel reducer
//     (Eager_AssignGroupBySize, paddle/fluid/distributed/collective/reducer.cc:48)
//   * communication watchdog: a background thread that tracks in-flight collectives by id, classifies
//     "never started" vs "started but not finished" timeouts and keeps the last completed task per group
//     (CommTaskManager::CommTaskLoop, paddle/phi/core/distributed/comm_task_manager.cc) — host-only, it
//     never blocks or touches the GPU; Python feeds it start/finish events and polls for verdicts
//   * reshard planner: placement transition -> sequence of collective steps
//     (paddle/phi/core/distributed/auto_parallel/reshard/*_reshard_function.cc)
//   * static argument checks for collectives (paddle/phi/core/distributed/check/static_check.cc:26-154)
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#define PD_EXPORT extern "C" __attribute__((visibility("default")))

namespace pdrt {

// ------------------------------------------------------------------------------------------- flags
static std::mutex g_flag_mu;
static std::map<std::string, std::string>& flags() {
  static std::map<std::string, std::string> f;
  return f;
}

// ------------------------------------------------------------------------------------------- watchdog
struct CommTask {
  int64_t id;
  int group;
  std::string name;
  int64_t bytes;
  std::chrono::steady_clock::time_point created, started;
  bool has_started = false, finished = false, reported = false;
};
struct Watchdog {
  std::mutex mu;
  std::condition_variable cv;
  std::map<int64_t, CommTask> tasks;
  std::map<int, std::string> last_done;   // group -> description of the last finished task
  std::vector<std::string> verdicts;      // timeout reports not yet fetched
  std::thread th;
  std::atomic<bool> stop{false};
  int timeout_ms = 1800000;
  int sleep_ms = 100;
  std::atomic<int64_t> next_id{1};
  void Loop() {
    while (!stop) {
      std::unique_lock<std::mutex> lk(mu);
      cv.wait_for(lk, std::chrono::milliseconds(sleep_ms));
      auto now = std::chrono::steady_clock::now();
      for (auto it = tasks.begin(); it != tasks.end();) {
        CommTask& t = it->second;
        if (t.finished) {
          last_done[t.group] = t.name + "#" + std::to_string(t.id);
          it = tasks.erase(it);
          continue;
        }
        auto ref = t.has_started ? t.started : t.created;
        auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(now - ref).count();
        if (!t.reported && ms > timeout_ms) {
          t.reported = true;
          std::string v = std::string(t.has_started ? "started-but-not-finished" : "timeout-not-started") +
                          " task=" + t.name + "#" + std::to_string(t.id) + " group=" + std::to_string(t.group) +
                          " bytes=" + std::to_string(t.bytes) + " waited_ms=" + std::to_string(ms) +
                          " last_done=" + (last_done.count(t.group) ? last_done[t.group] : std::string("none"));
          verdicts.push_back(v);
        }
        ++it;
      }
    }
  }
};
static Watchdog* g_wd = nullptr;

}  // namespace pdrt

using namespace pdrt;

// ------------------------------------------------------------------------------------------- flags API
PD_EXPORT void pd_flag_set(const char* name, const char* value) {
  std::lock_guard<std::mutex> g(g_flag_mu);
  flags()[name] = value;
}
// Returns the length of the value (copied into buf up to cap) or -1 if the flag is unknown and not in env.
PD_EXPORT int pd_flag_get(const char* name, char* buf, int cap) {
  std::lock_guard<std::mutex> g(g_flag_mu);
  auto it = flags().find(name);
  std::string v;
  if (it != flags().end()) {
    v = it->second;
  } else {
    const char* e = getenv(name);
    if (!e) return -1;
    v = e;
    flags()[name] = v;
  }
  int n = static_cast<int>(v.size());
  if (cap > 0) {
    int c = n < cap - 1 ? n : cap - 1;
    memcpy(buf, v.data(), c);
    buf[c] = 0;
  }
  return n;
}

// ------------------------------------------------------------------------------------------- bucketing
// sizes/dtypes are given in the order gradients become ready (reverse parameter order).  limits[0] caps the
// first group of each dtype, limits[last] every later one.  out_group[i] = group index of tensor i.
PD_EXPORT int pd_assign_group_by_size(const int64_t* sizes, const int* dtypes, int n, const int64_t* limits, int n_limits,
                                      int* out_group) {
  struct Open { std::vector<int> idx; int64_t bytes = 0; int limit_idx = 0; };
  std::map<int, Open> open;
  std::vector<std::vector<int>> groups;
  for (int i = 0; i < n; ++i) {
    Open& o = open[dtypes[i]];
    o.idx.push_back(i);
    o.bytes += sizes[i];
    int li = o.limit_idx < n_limits ? o.limit_idx : n_limits - 1;
    if (o.bytes >= limits[li]) {
      groups.push_back(o.idx);
      o.idx.clear();
      o.bytes = 0;
      o.limit_idx++;
    }
  }
  for (auto& kv : open)
    if (!kv.second.idx.empty()) groups.push_back(kv.second.idx);
  for (size_t g = 0; g < groups.size(); ++g)
    for (int i : groups[g]) out_group[i] = static_cast<int>(g);
  return static_cast<int>(groups.size());
}

// ------------------------------------------------------------------------------------------- watchdog API
PD_EXPORT void pd_watchdog_start(int timeout_ms, int sleep_ms) {
  if (g_wd) return;
  g_wd = new Watchdog();
  g_wd->timeout_ms = timeout_ms;
  g_wd->sleep_ms = sleep_ms;
  g_wd->th = std::thread([] { g_wd->Loop(); });
}
PD_EXPORT void pd_watchdog_stop() {
  if (!g_wd) return;
  g_wd->stop = true;
  g_wd->cv.notify_all();
  g_wd->th.join();
  delete g_wd;
  g_wd = nullptr;
}
PD_EXPORT int64_t pd_watchdog_task_create(int group, const char* name, int64_t bytes) {
  if (!g_wd) return 0;
  std::lock_guard<std::mutex> g(g_wd->mu);
  CommTask t;
  t.id = g_wd->next_id++;
  t.group = group;
  t.name = name;
  t.bytes = bytes;
  t.created = std::chrono::steady_clock::now();
  g_wd->tasks[t.id] = t;
  return t.id;
}
PD_EXPORT void pd_watchdog_task_started(int64_t id) {
  if (!g_wd) return;
  std::lock_guard<std::mutex> g(g_wd->mu);
  auto it = g_wd->tasks.find(id);
  if (it != g_wd->tasks.end()) {
    it->second.has_started = true;
    it->second.started = std::chrono::steady_clock::now();
  }
}
PD_EXPORT void pd_watchdog_task_finished(int64_t id) {
  if (!g_wd) return;
  std::lock_guard<std::mutex> g(g_wd->mu);
  auto it = g_wd->tasks.find(id);
  if (it != g_wd->tasks.end()) it->second.finished = true;
}
// Pops one timeout verdict into buf; returns its length, 0 if none.
PD_EXPORT int pd_watchdog_poll(char* buf, int cap) {
  if (!g_wd) return 0;
  std::lock_guard<std::mutex> g(g_wd->mu);
  if (g_wd->verdicts.empty()) return 0;
  std::string v = g_wd->verdicts.front();
  g_wd->verdicts.erase(g_wd->verdicts.begin());
  int c = static_cast<int>(v.size()) < cap - 1 ? static_cast<int>(v.size()) : cap - 1;
  memcpy(buf, v.data(), c);
  buf[c] = 0;
  return c;
}
PD_EXPORT int pd_watchdog_inflight() {
  if (!g_wd) return 0;
  std::lock_guard<std::mutex> g(g_wd->mu);
  int n = 0;
  for (auto& kv : g_wd->tasks) n += kv.second.finished ? 0 : 1;
  return n;
}

// ------------------------------------------------------------------------------------------- reshard planner
// Placement codes per mesh axis: -1 replicate, -2 partial(sum), >= 0 shard on that tensor dim.
// Writes steps as triples {op, mesh_axis, tensor_dim} into out (capacity cap triples); returns step count.
//   op: 1 all_gather (s->r)  2 all_reduce (p->r)  3 reduce_scatter (p->s)  4 slice (r->s)
//       5 all_to_all (s->s, dim change)           6 scale-to-partial (r->p: non-zero ranks zero their copy)
PD_EXPORT int pd_plan_reshard(const int* src, const int* dst, int mesh_ndim, int* out, int cap) {
  int n = 0;
  auto emit = [&](int op, int axis, int dim) {
    if (n < cap) { out[3 * n] = op; out[3 * n + 1] = axis; out[3 * n + 2] = dim; }
    ++n;
  };
  // resolve partial / shard sources first (innermost mesh axis first keeps shard order consistent)
  for (int a = mesh_ndim - 1; a >= 0; --a) {
    const int s = src[a], d = dst[a];
    if (s == d) continue;
    if (s == -2) {
      if (d == -1) emit(2, a, -1);
      else emit(3, a, d);
    } else if (s >= 0) {
      if (d == -1) emit(1, a, s);
      else if (d >= 0) emit(5, a, s * 1000 + d);
      else { emit(1, a, s); emit(6, a, -1); }
    }
  }
  for (int a = 0; a < mesh_ndim; ++a) {
    const int s = src[a], d = dst[a];
    if (s == -1 && d >= 0) emit(4, a, d);
    else if (s == -1 && d == -2) emit(6, a, -1);
  }
  return n;
}

// ------------------------------------------------------------------------------------------- static checks
// Returns 0 if ok, otherwise an error code: 1 rank out of range, 2 size not divisible, 3 size mismatch.
PD_EXPORT int pd_comm_static_check(int kind, int64_t in_numel, int64_t out_numel, int rank, int world, int root) {
  if (rank < 0 || rank >= world || (root >= world)) return 1;
  switch (kind) {
    case 0: return in_numel == out_numel ? 0 : 3;                                   // same-shape (all_reduce, broadcast)
    case 1: return out_numel == in_numel * world ? 0 : 3;                           // all_gather
    case 2: return (in_numel % world) ? 2 : (out_numel * world == in_numel ? 0 : 3);  // reduce_scatter / scatter
    case 3: return (in_numel % world) ? 2 : (in_numel == out_numel ? 0 : 3);        // all_to_all
    default: return 0;
  }
}

// ------------------------------------------------------------------------------------------- gradient reducer
// Bookkeeping of the data-parallel gradient reducer (EagerReducer, paddle/fluid/distributed/collective/reducer.cc:482:
// MarkVarReady :797, MarkGroupReady :944, FinalizeBackward :1040): which bucket a parameter belongs to, how many
// gradients of each bucket have arrived in the current backward pass, which bucket is complete and may be reduced,
// and - when backward ends - which buckets never completed (unused parameters).  The tensors themselves stay with the
// caller; this object only keeps the counters, so the per-gradient hook is one native call.
namespace {
struct Reducer {
  std::vector<int> bucket_of;      // parameter -> bucket
  std::vector<int> bucket_size;    // parameters per bucket
  std::vector<int> ready;          // gradients arrived per bucket in this backward
  std::vector<char> seen;          // parameter arrived in this backward
  std::vector<char> launched;      // bucket handed out for reduction in this backward
  bool in_backward = false;
  std::mutex mu;
};
}  // namespace

PD_EXPORT void* pd_reducer_create(const int* bucket_of_param, int n_params, int n_buckets) {
  auto* r = new Reducer();
  r->bucket_of.assign(bucket_of_param, bucket_of_param + n_params);
  r->bucket_size.assign(n_buckets, 0);
  for (int i = 0; i < n_params; ++i) {
    if (bucket_of_param[i] < 0 || bucket_of_param[i] >= n_buckets) {
      delete r;
      return nullptr;
    }
    r->bucket_size[bucket_of_param[i]]++;
  }
  r->ready.assign(n_buckets, 0);
  r->seen.assign(n_params, 0);
  r->launched.assign(n_buckets, 0);
  return r;
}
PD_EXPORT void pd_reducer_destroy(void* h) { delete static_cast<Reducer*>(h); }

// A gradient arrived.  Returns: bucket index (>= 0) when this arrival completed the bucket, -1 when the bucket is
// still incomplete, -2 when the parameter was already marked in this backward (a second use without no_sync),
// -3 for a bad index.  *first_of_backward is set to 1 for the first arrival of a backward pass: the caller queues its
// end-of-backward callback then (and not when a bucket happens to complete).
PD_EXPORT int pd_reducer_mark_ready(void* h, int param, int* first_of_backward) {
  auto* r = static_cast<Reducer*>(h);
  std::lock_guard<std::mutex> g(r->mu);
  if (param < 0 || param >= static_cast<int>(r->bucket_of.size())) return -3;
  *first_of_backward = r->in_backward ? 0 : 1;
  r->in_backward = true;
  if (r->seen[param]) return -2;
  r->seen[param] = 1;
  const int b = r->bucket_of[param];
  if (++r->ready[b] == r->bucket_size[b]) {
    r->launched[b] = 1;
    return b;
  }
  return -1;
}
// End of backward: writes the buckets that received some but not all gradients, or none at all, into out (capacity
// cap) and resets every counter for the next pass.  Returns how many there are.
PD_EXPORT int pd_reducer_finish(void* h, int* out, int cap) {
  auto* r = static_cast<Reducer*>(h);
  std::lock_guard<std::mutex> g(r->mu);
  int n = 0;
  for (size_t b = 0; b < r->ready.size(); ++b) {
    if (!r->launched[b]) {
      if (n < cap) out[n] = static_cast<int>(b);
      ++n;
    }
  }
  std::fill(r->ready.begin(), r->ready.end(), 0);
  std::fill(r->seen.begin(), r->seen.end(), 0);
  std::fill(r->launched.begin(), r->launched.end(), 0);
  r->in_backward = false;
  return n;
}
