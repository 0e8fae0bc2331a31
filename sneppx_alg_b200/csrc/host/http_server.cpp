// HTTP/1.1 front-end for the serving API: accept thread + worker pool, route table with {param} segments, Bearer
// authentication, per-route request / latency counters, static JSON routes and callback routes that hand the request
// to the embedding process (the Python serving engine registers its handlers as C callbacks). A callback receives the
// captured path parameters as a JSON object, plus the request's Authorization header under "_authorization" and the
// raw query string under "_query".
//
// Reference counterparts: net/http/http_server.c (routes with {param}, middleware chain, worker threads),
// net/http/http_auth.c (Bearer check), net/http/http_api.c:326-329 (/v1/health, /v1/models, /v1/models/{id},
// /v1/generate). The reference's /v1/generate returns pseudo-random tokens from a linear congruential generator; here
// the route calls into the engine that owns the GPU.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#define SX_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

// status is in/out: preset to 200. Returns the body length written to `out`, or -(needed) when `cap` is too small
// (the server retries once with a larger buffer).
typedef long long (*RouteCallback)(const char* method, const char* path, const char* params, const char* body,
                                   long long body_len, char* out, long long cap, int* status);

struct Route {
  std::string method;
  std::vector<std::string> segs;  // "{name}" segments capture
  bool is_public = false;
  std::string static_body;
  RouteCallback cb = nullptr;
  std::atomic<long long> hits{0};
  std::atomic<long long> micros{0};
};

std::vector<std::string> split_path(const std::string& p) {
  std::vector<std::string> v;
  std::string cur;
  for (char c : p) {
    if (c == '/') { if (!cur.empty()) v.push_back(cur); cur.clear(); }
    else cur += c;
  }
  if (!cur.empty()) v.push_back(cur);
  return v;
}

std::string json_escape(const std::string& s) {
  std::string o;
  for (unsigned char c : s) {
    if (c == '"' || c == '\\') { o += '\\'; o += (char)c; }
    else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); o += b; }
    else o += (char)c;
  }
  return o;
}

const char* reason(int st) {
  switch (st) {
    case 200: return "OK"; case 201: return "Created"; case 204: return "No Content"; case 400: return "Bad Request";
    case 401: return "Unauthorized"; case 403: return "Forbidden"; case 404: return "Not Found";
    case 405: return "Method Not Allowed"; case 413: return "Payload Too Large"; case 429: return "Too Many Requests";
    case 500: return "Internal Server Error"; case 503: return "Service Unavailable";
  }
  return "Status";
}

struct Server {
  int lfd = -1, port = 0;
  std::string token;
  size_t max_body = 8u << 20;
  std::atomic<bool> stop{false};
  std::thread acceptor;
  std::vector<std::thread> workers;
  std::mutex mu;
  std::condition_variable cv;
  std::deque<int> pending;
  std::vector<Route*> routes;
  std::atomic<long long> total{0}, rejected{0};

  ~Server() { for (auto* r : routes) delete r; }

  void respond(int fd, int st, const std::string& body, const char* ctype = "application/json") {
    std::ostringstream h;
    h << "HTTP/1.1 " << st << ' ' << reason(st) << "\r\nContent-Type: " << ctype << "\r\nContent-Length: " << body.size()
      << "\r\nConnection: close\r\n";
    if (st == 401) h << "WWW-Authenticate: Bearer\r\n";
    h << "\r\n";
    std::string head = h.str();
    ::send(fd, head.data(), head.size(), MSG_NOSIGNAL);
    if (!body.empty()) ::send(fd, body.data(), body.size(), MSG_NOSIGNAL);
  }

  std::string metrics() {
    std::ostringstream o;
    o << "{\"requests\":" << total.load() << ",\"rejected\":" << rejected.load() << ",\"routes\":[";
    bool first = true;
    for (auto* r : routes) {
      if (!first) o << ',';
      first = false;
      std::string pat;
      for (auto& s : r->segs) pat += "/" + s;
      long long n = r->hits.load();
      o << "{\"method\":\"" << r->method << "\",\"path\":\"" << json_escape(pat.empty() ? "/" : pat) << "\",\"hits\":" << n
        << ",\"mean_ms\":" << (n ? (double)r->micros.load() / n / 1000.0 : 0.0) << '}';
    }
    o << "]}";
    return o.str();
  }

  void handle(int fd) {
    timeval tv{5, 0};
    setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
    std::string buf;
    size_t head_end = std::string::npos;
    char tmp[8192];
    while (head_end == std::string::npos && buf.size() < 65536) {
      ssize_t k = ::recv(fd, tmp, sizeof tmp, 0);
      if (k <= 0) return;
      buf.append(tmp, (size_t)k);
      head_end = buf.find("\r\n\r\n");
    }
    if (head_end == std::string::npos) { respond(fd, 400, "{\"error\":\"header too large\"}"); return; }
    std::istringstream hs(buf.substr(0, head_end));
    std::string method, target, version, line;
    hs >> method >> target >> version;
    std::getline(hs, line);
    std::map<std::string, std::string> headers;
    while (std::getline(hs, line)) {
      if (!line.empty() && line.back() == '\r') line.pop_back();
      size_t c = line.find(':');
      if (c == std::string::npos) continue;
      std::string k = line.substr(0, c), v = line.substr(c + 1);
      for (auto& ch : k) ch = (char)tolower((unsigned char)ch);
      size_t b = v.find_first_not_of(' ');
      headers[k] = b == std::string::npos ? "" : v.substr(b);
    }
    size_t clen = 0;
    if (headers.count("content-length")) clen = (size_t)strtoull(headers["content-length"].c_str(), nullptr, 10);
    if (clen > max_body) { rejected++; respond(fd, 413, "{\"error\":\"body too large\"}"); return; }
    std::string body = buf.substr(head_end + 4);
    while (body.size() < clen) {
      ssize_t k = ::recv(fd, tmp, sizeof tmp, 0);
      if (k <= 0) return;
      body.append(tmp, (size_t)k);
    }
    body.resize(clen);
    std::string path = target.substr(0, target.find('?'));
    total++;
    if (method == "GET" && path == "/metrics/native") { respond(fd, 200, metrics()); return; }

    auto segs = split_path(path);
    Route* hit = nullptr;
    bool path_matched = false;
    std::string params = "{";
    for (auto* r : routes) {
      if (r->segs.size() != segs.size()) continue;
      std::string p = "{";
      bool ok = true;
      for (size_t i = 0; i < segs.size() && ok; ++i) {
        const std::string& s = r->segs[i];
        if (s.size() > 2 && s.front() == '{' && s.back() == '}') {
          if (p.size() > 1) p += ',';
          p += "\"" + s.substr(1, s.size() - 2) + "\":\"" + json_escape(segs[i]) + "\"";
        } else if (s != segs[i]) ok = false;
      }
      if (!ok) continue;
      path_matched = true;
      if (r->method == method) { hit = r; params = p; break; }
    }
    if (hit && hit->cb && headers.count("authorization")) {  // handlers that do their own per-user authorisation
      if (params.size() > 1) params += ',';
      params += "\"_authorization\":\"" + json_escape(headers["authorization"]) + "\"";
    }
    if (hit && hit->cb && target.find('?') != std::string::npos) {
      if (params.size() > 1) params += ',';
      params += "\"_query\":\"" + json_escape(target.substr(target.find('?') + 1)) + "\"";
    }
    params += "}";
    if (!hit) { rejected++; respond(fd, path_matched ? 405 : 404, path_matched ? "{\"error\":\"method not allowed\"}" : "{\"error\":\"not found\"}"); return; }
    if (!token.empty() && !hit->is_public) {
      auto it = headers.find("authorization");
      if (it == headers.end() || it->second != "Bearer " + token) { rejected++; respond(fd, 401, "{\"error\":\"missing or invalid bearer token\"}"); return; }
    }
    auto t0 = std::chrono::steady_clock::now();
    int st = 200;
    std::string out;
    if (hit->cb) {
      std::vector<char> ob(1 << 16);
      long long n = hit->cb(method.c_str(), path.c_str(), params.c_str(), body.data(), (long long)body.size(), ob.data(), (long long)ob.size(), &st);
      if (n < 0 && -n <= (4ll << 30)) {  // same worker thread asks again with room; the callee keeps its result
        ob.resize((size_t)-n);
        st = 200;
        n = hit->cb(method.c_str(), path.c_str(), params.c_str(), body.data(), (long long)body.size(), ob.data(), (long long)ob.size(), &st);
      }
      if (n < 0) { st = 500; out = "{\"error\":\"handler failed\"}"; }
      else out.assign(ob.data(), (size_t)n);
    } else out = hit->static_body;
    respond(fd, st, out);
    hit->hits++;
    hit->micros += std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
  }

  void worker() {
    for (;;) {
      int fd;
      {
        std::unique_lock<std::mutex> lk(mu);
        cv.wait(lk, [&] { return stop.load() || !pending.empty(); });
        if (pending.empty()) return;
        fd = pending.front();
        pending.pop_front();
      }
      handle(fd);
      ::close(fd);
    }
  }

  void accept_loop() {
    while (!stop) {
      pollfd p{lfd, POLLIN, 0};
      if (::poll(&p, 1, 100) <= 0) continue;
      int fd = ::accept(lfd, nullptr, nullptr);
      if (fd < 0) continue;
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
      std::lock_guard<std::mutex> lk(mu);
      pending.push_back(fd);
      cv.notify_one();
    }
  }
};

}  // namespace

// Routes must be added before sx_http_start. `token` empty disables authentication.
SX_EXPORT void* sx_http_create(const char* token, long long max_body) {
  auto* s = new Server;
  s->token = token ? token : "";
  if (max_body > 0) s->max_body = (size_t)max_body;
  return s;
}

SX_EXPORT int sx_http_add_route(void* h, const char* method, const char* pattern, int is_public, const char* static_body, RouteCallback cb) {
  auto* s = (Server*)h;
  auto* r = new Route;
  r->method = method;
  r->segs = split_path(pattern);
  r->is_public = is_public != 0;
  r->static_body = static_body ? static_body : "";
  r->cb = cb;
  s->routes.push_back(r);
  return (int)s->routes.size() - 1;
}

// `host`: dotted IPv4 address to bind ("0.0.0.0" for all interfaces); nullptr or "" binds the loopback interface.
SX_EXPORT int sx_http_start_on(void* h, const char* host, int port, int workers) {
  auto* s = (Server*)h;
  s->lfd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (s->lfd < 0) return -1;
  int one = 1;
  setsockopt(s->lfd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  if (host && *host && inet_pton(AF_INET, host, &a.sin_addr) != 1) { ::close(s->lfd); s->lfd = -1; return -1; }
  a.sin_port = htons((uint16_t)port);
  if (::bind(s->lfd, (sockaddr*)&a, sizeof a) || ::listen(s->lfd, 128)) { ::close(s->lfd); s->lfd = -1; return -1; }
  socklen_t l = sizeof a;
  getsockname(s->lfd, (sockaddr*)&a, &l);
  s->port = ntohs(a.sin_port);
  for (int i = 0; i < (workers < 1 ? 1 : workers); ++i) s->workers.emplace_back([s] { s->worker(); });
  s->acceptor = std::thread([s] { s->accept_loop(); });
  return s->port;
}

SX_EXPORT int sx_http_start(void* h, int port, int workers) { return sx_http_start_on(h, nullptr, port, workers); }

SX_EXPORT void sx_http_stop(void* h) {
  auto* s = (Server*)h;
  s->stop = true;
  if (s->acceptor.joinable()) s->acceptor.join();
  { std::lock_guard<std::mutex> lk(s->mu); s->cv.notify_all(); }
  for (auto& w : s->workers) if (w.joinable()) w.join();
  for (int fd : s->pending) ::close(fd);
  if (s->lfd >= 0) ::close(s->lfd);
  delete s;
}

SX_EXPORT long long sx_http_route_hits(void* h, int route) { return ((Server*)h)->routes[route]->hits.load(); }
