// CPU-rank distributed runtime: TCP ring all-reduce (scatter-reduce + all-gather, optional top-k compression with
// error feedback), versioned parameter sync (last writer wins by (version, node id)), Laplace noise for
// differentially-private sync, and a UDP heartbeat failure detector. It is the gloo-class fallback for hosts
// without GPUs and the vehicle for fault-injection tests (failures are made on the host: a node stops sending).
// C ABI names follow the reference's Rust runtime (net/distributed/src/lib.rs:881-1098: arix_dist_init / connect /
// all_reduce / ring_all_reduce / sync_params / add_noise / shutdown); heartbeat constants follow
// include/neural_core/kernel/heartbeat.h:39-40 (port 28700 + rank, magic 0x534E5048) and the SUSPECT / DEAD rules of
// kernel/distributed/heartbeat.c:189-210 (late => SUSPECT, three missed intervals => DEAD).
#include <arpa/inet.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <random>
#include <string>
#include <thread>
#include <vector>

namespace {

using Clock = std::chrono::steady_clock;
double now_s() { return std::chrono::duration<double>(Clock::now().time_since_epoch()).count(); }

struct Ring {
  int id = 0, world = 1;
  int listen_fd = -1, next_fd = -1, prev_fd = -1;
  std::vector<float> residual;  // error feedback of the top-k compressor
  int timeout_ms = 10000;
};
Ring g_ring;
std::mutex g_mu;

bool set_nodelay(int fd) {
  int one = 1;
  return setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one)) == 0;
}

// Full-duplex exchange: send `sn` bytes to next while receiving `rn` bytes from prev (poll-driven, bounded).
int exchange(const Ring& r, const void* sbuf, size_t sn, void* rbuf, size_t rn) {
  size_t so = 0, ro = 0;
  const double deadline = now_s() + r.timeout_ms / 1000.0;
  while (so < sn || ro < rn) {
    pollfd p[2];
    p[0] = {r.next_fd, (short)(so < sn ? POLLOUT : 0), 0};
    p[1] = {r.prev_fd, (short)(ro < rn ? POLLIN : 0), 0};
    const int rc = poll(p, 2, 200);
    if (rc < 0) return -1;
    if (now_s() > deadline) return -2;
    if (so < sn && (p[0].revents & POLLOUT)) {
      ssize_t k = send(r.next_fd, (const char*)sbuf + so, sn - so, MSG_NOSIGNAL | MSG_DONTWAIT);
      if (k > 0) so += (size_t)k;
      else if (k < 0 && errno != EAGAIN && errno != EWOULDBLOCK) return -3;
    }
    if (ro < rn && (p[1].revents & (POLLIN | POLLHUP))) {
      ssize_t k = recv(r.prev_fd, (char*)rbuf + ro, rn - ro, MSG_DONTWAIT);
      if (k > 0) ro += (size_t)k;
      else if (k == 0) return -4;  // peer closed
      else if (errno != EAGAIN && errno != EWOULDBLOCK) return -3;
    }
  }
  return 0;
}

void chunk_range(size_t n, int world, int c, size_t* b, size_t* e) {
  const size_t base = n / world, rem = n % world;
  *b = c * base + std::min<size_t>(c, rem);
  *e = *b + base + ((size_t)c < rem ? 1 : 0);
}

int ring_all_reduce(Ring& r, float* data, size_t n, bool average) {
  if (r.world == 1) return 0;
  size_t maxc = n / r.world + 1;
  std::vector<float> tmp(maxc);
  // scatter-reduce: after world-1 steps rank i owns the full sum of chunk (i+1) % world
  for (int s = 0; s < r.world - 1; ++s) {
    const int sc = ((r.id - s) % r.world + r.world) % r.world, rc = ((r.id - s - 1) % r.world + r.world) % r.world;
    size_t sb, se, rb, re;
    chunk_range(n, r.world, sc, &sb, &se);
    chunk_range(n, r.world, rc, &rb, &re);
    const int e = exchange(r, data + sb, (se - sb) * 4, tmp.data(), (re - rb) * 4);
    if (e) return e;
    for (size_t i = 0; i < re - rb; ++i) data[rb + i] += tmp[i];
  }
  // all-gather of the reduced chunks
  for (int s = 0; s < r.world - 1; ++s) {
    const int sc = ((r.id + 1 - s) % r.world + r.world) % r.world, rc = ((r.id - s) % r.world + r.world) % r.world;
    size_t sb, se, rb, re;
    chunk_range(n, r.world, sc, &sb, &se);
    chunk_range(n, r.world, rc, &rb, &re);
    const int e = exchange(r, data + sb, (se - sb) * 4, data + rb, (re - rb) * 4);
    if (e) return e;
  }
  if (average) {
    const float inv = 1.f / r.world;
    for (size_t i = 0; i < n; ++i) data[i] *= inv;
  }
  return 0;
}

// ------------------------------------------------------------------ heartbeat
constexpr uint32_t kHbMagic = 0x534E5048u;
enum { HB_ALIVE = 0, HB_SUSPECT = 1, HB_DEAD = 2 };
#pragma pack(push, 1)
struct HbMsg {
  uint32_t magic;
  int32_t rank, world, status;
  double ts;
};
#pragma pack(pop)

struct Heartbeat {
  int rank, world, base_port, interval_ms, timeout_ms;
  int fd = -1;
  std::atomic<bool> run{false}, send_enabled{true};
  std::vector<double> last_seen;
  std::vector<std::atomic<int>> status;
  std::thread th;
  std::mutex mu;
  Heartbeat(int r, int w) : rank(r), world(w), last_seen(w, 0.0), status(w) {
    for (auto& s : status) s = HB_ALIVE;
  }
  void loop() {
    double next_send = 0;
    while (run) {
      const double t = now_s();
      if (t >= next_send) {
        next_send = t + interval_ms / 1000.0;
        if (send_enabled) {
          HbMsg m{kHbMagic, rank, world, HB_ALIVE, t};
          for (int p = 0; p < world; ++p) {
            if (p == rank) continue;
            sockaddr_in a{};
            a.sin_family = AF_INET;
            a.sin_port = htons((uint16_t)(base_port + p));
            a.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
            sendto(fd, &m, sizeof(m), MSG_DONTWAIT, (sockaddr*)&a, sizeof(a));
          }
        }
      }
      pollfd pf{fd, POLLIN, 0};
      if (poll(&pf, 1, std::max(1, interval_ms / 4)) > 0) {
        HbMsg m;
        while (recv(fd, &m, sizeof(m), MSG_DONTWAIT) == (ssize_t)sizeof(m)) {
          if (m.magic == kHbMagic && m.rank >= 0 && m.rank < world) {
            std::lock_guard<std::mutex> lk(mu);
            last_seen[m.rank] = now_s();
          }
        }
      }
      const double t2 = now_s();
      std::lock_guard<std::mutex> lk(mu);
      for (int p = 0; p < world; ++p) {
        if (p == rank) continue;
        if (last_seen[p] == 0.0) last_seen[p] = t2;  // grace period starts at first check
        const double late = (t2 - last_seen[p]) * 1000.0;
        if (late > 3.0 * interval_ms && late > timeout_ms) status[p] = HB_DEAD;
        else if (late > timeout_ms) status[p] = HB_SUSPECT;
        else status[p] = HB_ALIVE;
      }
    }
  }
};

}  // namespace

extern "C" {

int arix_dist_init(int node_id, int world_size, int listen_port) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_ring = Ring();
  g_ring.id = node_id;
  g_ring.world = world_size;
  if (world_size == 1) return 0;
  int fd = socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return -1;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons((uint16_t)listen_port);
  a.sin_addr.s_addr = htonl(INADDR_ANY);
  if (bind(fd, (sockaddr*)&a, sizeof(a)) != 0 || listen(fd, 8) != 0) {
    close(fd);
    return -2;
  }
  g_ring.listen_fd = fd;
  return 0;
}

// addresses: comma separated "host:port" for every node in rank order. Connects to (id+1) % world and accepts the
// connection of (id-1) % world; bounded by timeout_ms.
int arix_dist_connect(const char* addresses, int timeout_ms) {
  Ring& r = g_ring;
  if (r.world == 1) return 0;
  r.timeout_ms = timeout_ms > 0 ? timeout_ms : 10000;
  std::vector<std::string> addrs;
  std::string s(addresses), cur;
  for (char c : s) {
    if (c == ',') { addrs.push_back(cur); cur.clear(); } else cur += c;
  }
  if (!cur.empty()) addrs.push_back(cur);
  if ((int)addrs.size() != r.world) return -1;
  const std::string& nx = addrs[(r.id + 1) % r.world];
  const size_t colon = nx.rfind(':');
  if (colon == std::string::npos) return -1;
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons((uint16_t)atoi(nx.substr(colon + 1).c_str()));
  if (inet_pton(AF_INET, nx.substr(0, colon).c_str(), &a.sin_addr) != 1) return -1;
  const double deadline = now_s() + r.timeout_ms / 1000.0;
  int fd = -1;
  while (now_s() < deadline) {
    fd = socket(AF_INET, SOCK_STREAM, 0);
    if (connect(fd, (sockaddr*)&a, sizeof(a)) == 0) break;
    close(fd);
    fd = -1;
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
  }
  if (fd < 0) return -2;
  set_nodelay(fd);
  r.next_fd = fd;
  pollfd pf{r.listen_fd, POLLIN, 0};
  const int left = (int)std::max(1.0, (deadline - now_s()) * 1000.0);
  if (poll(&pf, 1, left) <= 0) return -3;
  r.prev_fd = accept(r.listen_fd, nullptr, nullptr);
  if (r.prev_fd < 0) return -3;
  set_nodelay(r.prev_fd);
  return 0;
}

int arix_dist_ring_all_reduce(float* data, unsigned long long n, int topk) {
  Ring& r = g_ring;
  if (topk > 0 && (unsigned long long)topk < n) {
    // top-k sparsification with error feedback: what is not sent now is added back next time
    if (r.residual.size() != n) r.residual.assign(n, 0.f);
    std::vector<size_t> idx(n);
    for (size_t i = 0; i < n; ++i) {
      data[i] += r.residual[i];
      idx[i] = i;
    }
    std::nth_element(idx.begin(), idx.begin() + topk, idx.end(),
                     [&](size_t a, size_t b) { return std::fabs(data[a]) > std::fabs(data[b]); });
    std::vector<char> keep(n, 0);
    for (int i = 0; i < topk; ++i) keep[idx[i]] = 1;
    for (size_t i = 0; i < n; ++i) {
      r.residual[i] = keep[i] ? 0.f : data[i];
      if (!keep[i]) data[i] = 0.f;
    }
  }
  return ring_all_reduce(r, data, (size_t)n, true);
}
int arix_dist_all_reduce(float* data, unsigned long long n) { return arix_dist_ring_all_reduce(data, n, 0); }
int arix_dist_all_reduce_sum(float* data, unsigned long long n) { return ring_all_reduce(g_ring, data, (size_t)n, false); }

// Every node ends up with the parameters of the node holding the highest (version, node id); *version is updated.
int arix_dist_sync_params(float* data, unsigned long long n, unsigned long long* version) {
  Ring& r = g_ring;
  if (r.world == 1) return 0;
  struct Tag { unsigned long long version; int node; int pad; } best{*version, r.id, 0};
  std::vector<float> cur(data, data + n), in((size_t)n);
  for (int s = 0; s < r.world - 1; ++s) {
    Tag got{};
    int e = exchange(r, &best, sizeof(best), &got, sizeof(got));
    if (e) return e;
    e = exchange(r, cur.data(), n * 4, in.data(), n * 4);
    if (e) return e;
    if (got.version > best.version || (got.version == best.version && got.node > best.node)) {
      best = got;
      cur.swap(in);
    }
  }
  memcpy(data, cur.data(), n * 4);
  *version = best.version;
  return 0;
}

// Laplace(0, scale) noise (differentially-private sync)
int arix_dist_add_noise(float* data, unsigned long long n, float scale, unsigned long long seed) {
  std::mt19937_64 rng(seed);
  std::uniform_real_distribution<double> u(-0.5, 0.5);
  for (unsigned long long i = 0; i < n; ++i) {
    const double x = u(rng);
    data[i] += (float)(-scale * (x < 0 ? -1.0 : 1.0) * std::log(1.0 - 2.0 * std::fabs(x)));
  }
  return 0;
}

int arix_dist_shutdown() {
  Ring& r = g_ring;
  for (int* fd : {&r.next_fd, &r.prev_fd, &r.listen_fd})
    if (*fd >= 0) { close(*fd); *fd = -1; }
  return 0;
}

// ---- heartbeat
void* sx_hb_create(int rank, int world, int base_port, int interval_ms, int timeout_ms) {
  Heartbeat* h = new Heartbeat(rank, world);
  h->base_port = base_port > 0 ? base_port : 28700;
  h->interval_ms = interval_ms;
  h->timeout_ms = timeout_ms;
  h->fd = socket(AF_INET, SOCK_DGRAM, 0);
  int fl = fcntl(h->fd, F_GETFL, 0);
  fcntl(h->fd, F_SETFL, fl | O_NONBLOCK);
  int one = 1;
  setsockopt(h->fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons((uint16_t)(h->base_port + rank));
  a.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  if (bind(h->fd, (sockaddr*)&a, sizeof(a)) != 0) {
    close(h->fd);
    delete h;
    return nullptr;
  }
  return h;
}
void sx_hb_start(void* p) {
  Heartbeat* h = static_cast<Heartbeat*>(p);
  h->run = true;
  h->th = std::thread([h] { h->loop(); });
}
int sx_hb_status(void* p, int rank) { return static_cast<Heartbeat*>(p)->status[rank].load(); }
void sx_hb_set_send_enabled(void* p, int on) { static_cast<Heartbeat*>(p)->send_enabled = on != 0; }
void sx_hb_stop(void* p) {
  Heartbeat* h = static_cast<Heartbeat*>(p);
  h->run = false;
  if (h->th.joinable()) h->th.join();
  close(h->fd);
  delete h;
}

}  // extern "C"
