// Work-stealing thread pool with futures, task groups, named workloads, parallel_for and parallel_reduce.
//
// Each worker owns a deque: it pushes and pops its own tasks at the back (LIFO keeps caches warm) and, when empty,
// steals from the FRONT of another worker's deque (the oldest, typically largest, piece of work). Tasks submitted
// from outside the pool are dealt round-robin over the deques; tasks submitted from a worker thread go to that
// worker's own deque, which is what makes recursive divide-and-conquer (parallel_for splitting ranges in halves)
// balance itself. A future is a one-shot result slot with a condition variable; a task group counts outstanding
// tasks and waits with an optional timeout; a pool worker that waits HELPS (it runs queued tasks itself, so a task may
// wait for a group it spawned without dead-locking the pool); a workload is a named task list with progress and
// cancellation. Behavioural counterpart of the reference's pool and dispatch layer
// (kernel/thread/threadpool.c:86-148,309 futures + stealing; kernel/thread/workload_dispatch.c:36-160 workloads and
// task groups; include/neural_core/kernel/concurrent_workload_dispatch.h:46-170 parallel_for / parallel_reduce).
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

struct Future {
  std::mutex mu;
  std::condition_variable cv;
  bool ready = false;
  void* result = nullptr;
};

struct Group {
  std::atomic<long long> pending{0};
  std::atomic<long long> completed{0};
  std::atomic<bool> cancelled{false};
  std::mutex mu;
  std::condition_variable cv;
};

struct Task {
  std::function<void()> fn;
};

struct WorkerQueue {
  std::mutex mu;
  std::deque<Task> dq;
};

struct Pool;
thread_local Pool* tl_pool = nullptr;
thread_local int tl_index = -1;

struct Pool {
  std::vector<std::thread> threads;
  std::vector<WorkerQueue*> queues;
  std::mutex sleep_mu;
  std::condition_variable sleep_cv;
  std::atomic<long long> queued{0};      // tasks sitting in deques
  std::atomic<long long> in_flight{0};   // queued + running
  std::atomic<long long> steals{0};
  std::atomic<long long> executed{0};
  std::atomic<unsigned> rr{0};
  std::atomic<bool> stop{false};
  std::mutex idle_mu;
  std::condition_variable idle_cv;

  explicit Pool(int n) {
    if (n <= 0) n = (int)std::thread::hardware_concurrency();
    if (n <= 0) n = 1;
    for (int i = 0; i < n; ++i) queues.push_back(new WorkerQueue());
    for (int i = 0; i < n; ++i) threads.emplace_back([this, i] { run(i); });
  }
  ~Pool() {
    stop.store(true);
    {
      std::lock_guard<std::mutex> lk(sleep_mu);
    }
    sleep_cv.notify_all();
    for (auto& t : threads) t.join();
    for (auto* q : queues) delete q;
  }

  void push(Task t) {
    const bool own = tl_pool == this && tl_index >= 0;
    int target = own ? tl_index : (int)(rr.fetch_add(1) % queues.size());
    in_flight.fetch_add(1);
    {
      // a worker's own spawn goes to the back (it pops there: newest first, depth first); a submission from
      // outside goes to the front, so outside submissions to one deque run in the order they were made
      std::lock_guard<std::mutex> lk(queues[target]->mu);
      if (own) queues[target]->dq.push_back(std::move(t));
      else queues[target]->dq.push_front(std::move(t));
    }
    queued.fetch_add(1);
    {
      std::lock_guard<std::mutex> lk(sleep_mu);
    }
    sleep_cv.notify_one();
  }

  bool pop_local(int i, Task& out) {
    std::lock_guard<std::mutex> lk(queues[i]->mu);
    if (queues[i]->dq.empty()) return false;
    out = std::move(queues[i]->dq.back());
    queues[i]->dq.pop_back();
    return true;
  }
  bool steal(int thief, Task& out) {
    const int n = (int)queues.size();
    for (int k = 1; k <= n; ++k) {
      const int v = (thief + k) % n;
      if (v == thief) continue;
      std::lock_guard<std::mutex> lk(queues[v]->mu);
      if (!queues[v]->dq.empty()) {
        out = std::move(queues[v]->dq.front());
        queues[v]->dq.pop_front();
        steals.fetch_add(1);
        return true;
      }
    }
    return false;
  }
  // Take any task: own deque first (workers), then steal. `self` < 0 for threads outside the pool.
  bool take(int self, Task& out) {
    if (self >= 0 && pop_local(self, out)) return true;
    return steal(self >= 0 ? self : 0, out) || (self < 0 && pop_local(0, out));
  }
  void execute(Task& t) {
    queued.fetch_sub(1);
    t.fn();
    executed.fetch_add(1);
    if (in_flight.fetch_sub(1) == 1) {
      std::lock_guard<std::mutex> lk(idle_mu);
      idle_cv.notify_all();
    }
  }
  void run(int i) {
    tl_pool = this;
    tl_index = i;
    Task t;
    while (true) {
      if (take(i, t)) {
        execute(t);
        t.fn = nullptr;
        continue;
      }
      std::unique_lock<std::mutex> lk(sleep_mu);
      if (stop.load()) break;
      if (queued.load() > 0) continue;
      sleep_cv.wait_for(lk, std::chrono::milliseconds(50));
      if (stop.load() && queued.load() == 0) break;
    }
  }
  // Run tasks on the calling thread until `done()` holds (or the deadline passes). Returns done().
  template <class Pred>
  bool help_until(Pred done, int timeout_ms) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms < 0 ? 0 : timeout_ms);
    const int self = (tl_pool == this) ? tl_index : -1;
    Task t;
    while (!done()) {
      // only a pool worker helps (it would otherwise block a thread the waited-for tasks may need); a thread from
      // outside just waits, so its timeout is honoured even when the queued tasks are long
      if (self >= 0 && take(self, t)) {
        execute(t);
        t.fn = nullptr;
        continue;
      }
      if (timeout_ms >= 0 && std::chrono::steady_clock::now() >= deadline) return done();
      std::this_thread::sleep_for(std::chrono::microseconds(self >= 0 ? 50 : 200));
    }
    return true;
  }
  void wait_idle() {
    help_until([this] { return in_flight.load() == 0; }, -1);
  }
};

void group_submit(Pool* p, Group* g, std::function<void()> fn) {
  g->pending.fetch_add(1);
  p->push(Task{[g, fn] {
    if (!g->cancelled.load()) fn();
    g->completed.fetch_add(1);
    if (g->pending.fetch_sub(1) == 1) {
      std::lock_guard<std::mutex> lk(g->mu);
      g->cv.notify_all();
    }
  }});
}

void range_split(Pool* p, Group* g, long long lo, long long hi, long long grain,
                 const std::function<void(long long, long long)>& body) {
  // split in halves; the right half is pushed (stealable), the left half continues on this thread
  while (hi - lo > grain) {
    const long long mid = lo + (hi - lo) / 2;
    group_submit(p, g, [p, g, mid, hi, grain, body] { range_split(p, g, mid, hi, grain, body); });
    hi = mid;
  }
  if (hi > lo) body(lo, hi);
}

struct Workload {
  struct Item {
    std::string name;
    void (*fn)(void*);
    void* arg;
  };
  std::vector<Item> items;
  size_t max_tasks;
  Group group;
  Pool* pool = nullptr;
  bool own_pool = false;
};

}  // namespace

extern "C" {

typedef void (*sx_wp_task_fn)(void*);
typedef void* (*sx_wp_result_fn)(void*);
typedef void (*sx_wp_range_fn)(long long, long long, void*);
typedef void (*sx_wp_reduce_fn)(long long, long long, void*, void*);
typedef void (*sx_wp_combine_fn)(void*, const void*);

void* sx_wp_create(int threads) { return new Pool(threads); }
void sx_wp_destroy(void* h) { delete static_cast<Pool*>(h); }
int sx_wp_num_threads(void* h) { return (int)static_cast<Pool*>(h)->threads.size(); }
int sx_wp_default_count(void) {
  const int n = (int)std::thread::hardware_concurrency();
  return n > 0 ? n : 1;
}
// out3: tasks executed, steals, tasks currently queued
void sx_wp_stats(void* h, long long* out3) {
  Pool* p = static_cast<Pool*>(h);
  out3[0] = p->executed.load();
  out3[1] = p->steals.load();
  out3[2] = p->queued.load();
}
int sx_wp_submit(void* h, sx_wp_task_fn fn, void* arg) {
  if (!h || !fn) return -1;
  static_cast<Pool*>(h)->push(Task{[fn, arg] { fn(arg); }});
  return 0;
}
void sx_wp_wait(void* h) { static_cast<Pool*>(h)->wait_idle(); }

// ---- futures
void* sx_wp_future_create(void) { return new Future(); }
void sx_wp_future_destroy(void* f) { delete static_cast<Future*>(f); }
void sx_wp_future_set_result(void* f, void* result) {
  Future* fu = static_cast<Future*>(f);
  {
    std::lock_guard<std::mutex> lk(fu->mu);
    fu->result = result;
    fu->ready = true;
  }
  fu->cv.notify_all();
}
int sx_wp_future_is_ready(void* f) {
  Future* fu = static_cast<Future*>(f);
  std::lock_guard<std::mutex> lk(fu->mu);
  return fu->ready ? 1 : 0;
}
// 1 when ready, 0 on timeout (timeout_ms < 0: wait for ever)
int sx_wp_future_wait(void* f, int timeout_ms) {
  Future* fu = static_cast<Future*>(f);
  std::unique_lock<std::mutex> lk(fu->mu);
  if (timeout_ms < 0) {
    fu->cv.wait(lk, [fu] { return fu->ready; });
    return 1;
  }
  return fu->cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), [fu] { return fu->ready; }) ? 1 : 0;
}
void* sx_wp_future_get_result(void* f) {
  sx_wp_future_wait(f, -1);
  return static_cast<Future*>(f)->result;
}
// The task's return value becomes the future's result.
int sx_wp_submit_future(void* h, sx_wp_result_fn fn, void* arg, void* fut) {
  if (!h || !fn || !fut) return -1;
  static_cast<Pool*>(h)->push(Task{[fn, arg, fut] { sx_wp_future_set_result(fut, fn(arg)); }});
  return 0;
}

// ---- task groups
void* sx_wp_group_create(void) { return new Group(); }
void sx_wp_group_destroy(void* g) { delete static_cast<Group*>(g); }
int sx_wp_group_add(void* h, void* g, sx_wp_task_fn fn, void* arg) {
  if (!h || !g || !fn) return -1;
  group_submit(static_cast<Pool*>(h), static_cast<Group*>(g), [fn, arg] { fn(arg); });
  return 0;
}
// Wait (helping to run tasks) until every task of the group has finished; 1 done, 0 timed out.
int sx_wp_group_wait(void* h, void* g, int timeout_ms) {
  Group* gr = static_cast<Group*>(g);
  return static_cast<Pool*>(h)->help_until([gr] { return gr->pending.load() == 0; }, timeout_ms) ? 1 : 0;
}
// Tasks of the group that have not started yet are skipped (they still count as completed).
void sx_wp_group_cancel(void* g) { static_cast<Group*>(g)->cancelled.store(true); }
long long sx_wp_group_completed(void* g) { return static_cast<Group*>(g)->completed.load(); }

// ---- ranges
void sx_wp_parallel_for(void* h, long long start, long long end, long long grain, sx_wp_range_fn fn, void* arg) {
  if (end <= start) return;
  Pool* p = static_cast<Pool*>(h);
  if (grain <= 0) {
    const long long parts = (long long)p->threads.size() * 4;
    grain = (end - start + parts - 1) / parts;
    if (grain < 1) grain = 1;
  }
  Group g;
  std::function<void(long long, long long)> body = [fn, arg](long long a, long long b) { fn(a, b, arg); };
  g.pending.fetch_add(1);
  range_split(p, &g, start, end, grain, body);
  g.pending.fetch_sub(1);
  p->help_until([&g] { return g.pending.load() == 0; }, -1);
}
// result starts as a copy of init; each chunk reduces into its own copy of init; copies are combined in index order.
void sx_wp_parallel_reduce(void* h, long long start, long long end, const void* init, size_t elem_size,
                           sx_wp_reduce_fn reduce_fn, sx_wp_combine_fn combine_fn, void* result, void* arg) {
  std::memcpy(result, init, elem_size);
  if (end <= start) return;
  Pool* p = static_cast<Pool*>(h);
  const long long parts = std::min<long long>(end - start, (long long)p->threads.size() * 4);
  const long long step = (end - start + parts - 1) / parts;
  std::vector<std::vector<unsigned char>> partial((size_t)parts, std::vector<unsigned char>(elem_size));
  Group g;
  for (long long i = 0; i < parts; ++i) {
    std::memcpy(partial[(size_t)i].data(), init, elem_size);
    const long long a = start + i * step, b = std::min(end, a + step);
    void* dst = partial[(size_t)i].data();
    group_submit(p, &g, [reduce_fn, a, b, arg, dst] {
      if (b > a) reduce_fn(a, b, arg, dst);
    });
  }
  p->help_until([&g] { return g.pending.load() == 0; }, -1);
  for (long long i = 0; i < parts; ++i) combine_fn(result, partial[(size_t)i].data());
}

// ---- named workloads
void* sx_wp_workload_create(long long max_tasks) {
  Workload* w = new Workload();
  w->max_tasks = (size_t)(max_tasks > 0 ? max_tasks : 0);
  return w;
}
void sx_wp_workload_destroy(void* wl) {
  Workload* w = static_cast<Workload*>(wl);
  if (w->pool && w->own_pool) {
    w->pool->wait_idle();
    delete w->pool;
  }
  delete w;
}
int sx_wp_workload_add_task(void* wl, const char* name, sx_wp_task_fn fn, void* arg) {
  Workload* w = static_cast<Workload*>(wl);
  if (!fn || (w->max_tasks && w->items.size() >= w->max_tasks)) return -1;
  w->items.push_back({name ? name : "", fn, arg});
  return (int)w->items.size() - 1;
}
// Runs the tasks on `pool` (or on a private pool of num_threads when pool is null).
int sx_wp_workload_submit(void* wl, void* pool, int num_threads) {
  Workload* w = static_cast<Workload*>(wl);
  if (w->pool) return -1;
  w->pool = pool ? static_cast<Pool*>(pool) : new Pool(num_threads);
  w->own_pool = pool == nullptr;
  for (auto& it : w->items) group_submit(w->pool, &w->group, [it] { it.fn(it.arg); });
  return 0;
}
int sx_wp_workload_wait(void* wl, int timeout_ms) {
  Workload* w = static_cast<Workload*>(wl);
  if (!w->pool) return -1;
  return w->pool->help_until([w] { return w->group.pending.load() == 0; }, timeout_ms) ? 1 : 0;
}
long long sx_wp_workload_num_completed(void* wl) { return static_cast<Workload*>(wl)->group.completed.load(); }
int sx_wp_workload_cancel(void* wl) {
  static_cast<Workload*>(wl)->group.cancelled.store(true);
  return 0;
}
const char* sx_wp_workload_task_name(void* wl, int i) {
  Workload* w = static_cast<Workload*>(wl);
  return (i >= 0 && (size_t)i < w->items.size()) ? w->items[(size_t)i].name.c_str() : "";
}

}  // extern "C"
