// Serving batch core in C++: request queue with size / timeout batching and FCFS or priority order, latency reservoir
// with percentiles and requests-per-second, weighted A/B routing by request-id hash, circuit breaker. This is the
// host-side logic of the reference's C serving engine and circuit breaker (net/http/serving_engine.c,
// include/neural_core/network/circuit_breaker.h); the Python control plane (serving/serving_engine.py) mirrors it.
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <queue>
#include <string>
#include <vector>

namespace {
double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
struct Item {
  long long id;
  int priority;
  double t;
  long long seq;
};
struct Cmp {
  bool operator()(const Item& a, const Item& b) const {
    if (a.priority != b.priority) return a.priority > b.priority;  // lower value first
    return a.seq > b.seq;
  }
};
struct Core {
  std::mutex mu;
  std::priority_queue<Item, std::vector<Item>, Cmp> q;
  long long seq = 0;
  int max_batch = 32;
  double timeout_s = 0.002;
  std::vector<double> lat;
  size_t lat_cap = 4096, lat_pos = 0;
  long long requests = 0, errors = 0;
  double start = now_s();
  // circuit breaker
  int fail_threshold = 5, consecutive_fail = 0, state = 0;  // 0 closed, 1 open, 2 half-open
  double open_until = 0, cooldown_s = 1.0;
};
uint64_t fnv1a(const char* s) {
  uint64_t h = 1469598103934665603ull;
  for (; *s; ++s) { h ^= (unsigned char)*s; h *= 1099511628211ull; }
  return h;
}
}  // namespace

extern "C" {
void* sx_sc_create(int max_batch, double timeout_ms) {
  Core* c = new Core();
  c->max_batch = max_batch;
  c->timeout_s = timeout_ms / 1000.0;
  return c;
}
void sx_sc_destroy(void* h) { delete static_cast<Core*>(h); }
void sx_sc_submit(void* h, long long id, int priority) {
  Core* c = static_cast<Core*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  c->q.push({id, priority, now_s(), c->seq++});
}
// Fills out[] with up to max_batch ids when the batch is full or the oldest request waited longer than the timeout.
int sx_sc_next_batch(void* h, long long* out, int cap, int force) {
  Core* c = static_cast<Core*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  if (c->q.empty()) return 0;
  // oldest arrival among queued items decides the timeout
  std::vector<Item> items;
  double oldest = 1e300;
  while (!c->q.empty()) { items.push_back(c->q.top()); oldest = std::min(oldest, items.back().t); c->q.pop(); }
  const bool fire = force || (int)items.size() >= c->max_batch || now_s() - oldest >= c->timeout_s;
  int n = 0;
  for (auto& it : items) {
    if (fire && n < c->max_batch && n < cap) out[n++] = it.id;
    else c->q.push(it);
  }
  return n;
}
int sx_sc_pending(void* h) {
  Core* c = static_cast<Core*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  return (int)c->q.size();
}
void sx_sc_record(void* h, double latency_s, int ok) {
  Core* c = static_cast<Core*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  c->requests++;
  if (!ok) c->errors++;
  if (c->lat.size() < c->lat_cap) c->lat.push_back(latency_s);
  else { c->lat[c->lat_pos] = latency_s; c->lat_pos = (c->lat_pos + 1) % c->lat_cap; }
  if (ok) { c->consecutive_fail = 0; if (c->state == 2) c->state = 0; }
  else if (++c->consecutive_fail >= c->fail_threshold || c->state == 2) { c->state = 1; c->open_until = now_s() + c->cooldown_s; }
}
// out: p50, p95, p99, rps, requests, errors
void sx_sc_metrics(void* h, double* out) {
  Core* c = static_cast<Core*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  std::vector<double> s(c->lat);
  std::sort(s.begin(), s.end());
  auto pct = [&](double q) { return s.empty() ? 0.0 : s[std::min(s.size() - 1, (size_t)(q * (s.size() - 1) + 0.5))]; };
  out[0] = pct(0.5); out[1] = pct(0.95); out[2] = pct(0.99);
  out[3] = c->requests / std::max(1e-9, now_s() - c->start);
  out[4] = (double)c->requests; out[5] = (double)c->errors;
}
// weights[n] -> index chosen deterministically from the request id
int sx_sc_route(const char* request_id, const double* weights, int n) {
  double tot = 0;
  for (int i = 0; i < n; ++i) tot += weights[i];
  if (tot <= 0) return -1;
  const double x = (double)(fnv1a(request_id) % 1000003) / 1000003.0 * tot;
  double acc = 0;
  for (int i = 0; i < n; ++i) { acc += weights[i]; if (x < acc) return i; }
  return n - 1;
}
void sx_sc_breaker_config(void* h, int fail_threshold, double cooldown_ms) {
  Core* c = static_cast<Core*>(h);
  c->fail_threshold = fail_threshold;
  c->cooldown_s = cooldown_ms / 1000.0;
}
// 1 when a request may pass (closed, or half-open probe after the cool-down)
int sx_sc_breaker_allow(void* h) {
  Core* c = static_cast<Core*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  if (c->state == 1 && now_s() >= c->open_until) c->state = 2;
  return c->state != 1;
}
int sx_sc_breaker_state(void* h) { return static_cast<Core*>(h)->state; }
}
