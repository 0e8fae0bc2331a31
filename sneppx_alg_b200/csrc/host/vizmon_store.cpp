// Metric store of the monitoring dashboard: named scalar series in fixed-size rings (oldest samples drop), per-series
// summaries (count, min, max, mean, last, p50 / p95 of the retained window), timeline spans, and incremental reads:
// every sample gets a global sequence number, and a reader asks for "everything after sequence s", which is what the
// live WebSocket feed sends every tick. Output is JSON text written into a caller buffer.
// Counterpart of the C store inside the reference's dashboard server (net/http/vizmon.c: scalar series, timeline,
// JSON endpoints).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace {

struct Sample {
  uint64_t seq;
  long long step;
  double value, ts;
};
struct Series {
  std::vector<Sample> ring;
  size_t head = 0, count = 0;
  uint64_t total = 0;
};
struct Span {
  uint64_t seq;
  std::string name;
  double start, end;
};
struct Store {
  std::mutex mu;
  size_t capacity;
  std::map<std::string, Series> series;
  std::vector<Span> spans;
  size_t span_head = 0, span_count = 0;
  uint64_t seq = 0;
};

void json_escape(std::string& out, const std::string& s) {
  for (char c : s) {
    if (c == '"' || c == '\\') { out += '\\'; out += c; }
    else if ((unsigned char)c < 0x20) { char b[8]; std::snprintf(b, sizeof b, "\\u%04x", c); out += b; }
    else out += c;
  }
}
void num(std::string& out, double v) {
  char b[40];
  if (std::isfinite(v)) std::snprintf(b, sizeof b, "%.9g", v);
  else std::snprintf(b, sizeof b, "null");
  out += b;
}
template <class F>
void for_each_sample(const Series& s, F f) {
  const size_t cap = s.ring.size();
  for (size_t i = 0; i < s.count; ++i) f(s.ring[(s.head + cap - s.count + i) % cap]);
}
long long emit(const std::string& js, char* buf, size_t cap) {
  if (js.size() + 1 > cap) return -(long long)(js.size() + 1);
  std::memcpy(buf, js.c_str(), js.size() + 1);
  return (long long)js.size();
}

}  // namespace

extern "C" {

void* sx_viz_create(size_t capacity) {
  Store* s = new Store();
  s->capacity = capacity ? capacity : 1024;
  s->spans.resize(s->capacity);
  return s;
}
void sx_viz_destroy(void* h) { delete static_cast<Store*>(h); }
// returns the sample's global sequence number
unsigned long long sx_viz_scalar(void* h, const char* name, long long step, double value, double ts) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  Series& se = s->series[name];
  if (se.ring.empty()) se.ring.resize(s->capacity);
  if (step < 0) step = (long long)se.total;
  se.ring[se.head] = Sample{++s->seq, step, value, ts};
  se.head = (se.head + 1) % se.ring.size();
  se.count = std::min(se.count + 1, se.ring.size());
  se.total++;
  return s->seq;
}
unsigned long long sx_viz_span(void* h, const char* name, double start, double end) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  s->spans[s->span_head] = Span{++s->seq, name, start, end};
  s->span_head = (s->span_head + 1) % s->spans.size();
  s->span_count = std::min(s->span_count + 1, s->spans.size());
  return s->seq;
}
unsigned long long sx_viz_sequence(void* h) { return static_cast<Store*>(h)->seq; }
// out8: retained count, total count, min, max, mean, last, p50, p95. Returns 0 when the series does not exist.
int sx_viz_summary(void* h, const char* name, double* out8) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  auto it = s->series.find(name);
  if (it == s->series.end() || it->second.count == 0) return 0;
  std::vector<double> v;
  double sum = 0, last = 0;
  for_each_sample(it->second, [&](const Sample& x) { v.push_back(x.value); sum += x.value; last = x.value; });
  std::sort(v.begin(), v.end());
  auto pct = [&](double q) { return v[std::min(v.size() - 1, (size_t)(q * (double)v.size()))]; };
  out8[0] = (double)v.size(); out8[1] = (double)it->second.total; out8[2] = v.front(); out8[3] = v.back();
  out8[4] = sum / (double)v.size(); out8[5] = last; out8[6] = pct(0.5); out8[7] = pct(0.95);
  return 1;
}
// {"seq": N, "scalars": {name: [[step, value, ts], ...]}, "spans": [{"name", "start", "end"}, ...]} restricted to
// entries with sequence number > after. Returns the JSON length, or -(bytes needed) when buf is too small.
long long sx_viz_snapshot(void* h, unsigned long long after, char* buf, size_t cap) {
  Store* s = static_cast<Store*>(h);
  std::string js;
  {
    std::lock_guard<std::mutex> lk(s->mu);
    js = "{\"seq\": " + std::to_string(s->seq) + ", \"scalars\": {";
    bool first_series = true;
    for (auto& kv : s->series) {
      std::string body;
      bool first = true;
      for_each_sample(kv.second, [&](const Sample& x) {
        if (x.seq <= after) return;
        body += first ? "[" : ", [";
        first = false;
        body += std::to_string(x.step) + ", ";
        num(body, x.value);
        body += ", ";
        num(body, x.ts);
        body += "]";
      });
      if (first && after > 0) continue;      // nothing new in this series
      js += first_series ? "\"" : ", \"";
      first_series = false;
      json_escape(js, kv.first);
      js += "\": [" + body + "]";
    }
    js += "}, \"spans\": [";
    bool first = true;
    const size_t capn = s->spans.size();
    for (size_t i = 0; i < s->span_count; ++i) {
      const Span& sp = s->spans[(s->span_head + capn - s->span_count + i) % capn];
      if (sp.seq <= after) continue;
      js += first ? "{\"name\": \"" : ", {\"name\": \"";
      first = false;
      json_escape(js, sp.name);
      js += "\", \"start\": ";
      num(js, sp.start);
      js += ", \"end\": ";
      num(js, sp.end);
      js += "}";
    }
    js += "]}";
  }
  return emit(js, buf, cap);
}
long long sx_viz_series_names(void* h, char* buf, size_t cap) {
  Store* s = static_cast<Store*>(h);
  std::string js = "[";
  {
    std::lock_guard<std::mutex> lk(s->mu);
    bool first = true;
    for (auto& kv : s->series) {
      js += first ? "\"" : ", \"";
      first = false;
      json_escape(js, kv.first);
      js += "\"";
    }
  }
  js += "]";
  return emit(js, buf, cap);
}

}  // extern "C"
