// Host-side network components: rank topology with routes, framed TCP messages with tensor transfer, a rendezvous
// coordinator (register / rank / barrier / all-gather / relayed tensor send-recv with a shared token), a Raft core
// (election, log replication, commit) driven by explicit ticks and message delivery, health checks, and the
// WebSocket / MQTT wire codecs.
//
// Reference counterparts: net/topology.c (ring / tree / graph and route search), net/socket/socket_comm.c (framed
// send / recv and tensor transfer), net/grpc/grpc_service.c (coordinator verbs), net/consensus/raft.c (API only; the
// bodies there return 0), net/monitoring/health_check.c, net/websocket/websocket_client.c, net/mqtt/mqtt_client.c.
// None of this is on the GPU path: NCCL and the peer-memory kernels carry tensors between GPUs; these carry control
// traffic and CPU-rank fallbacks.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <queue>
#include <string>
#include <thread>
#include <vector>

#define SX_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

// ---------------------------------------------------------------------------------------------------------------
// Topology
// ---------------------------------------------------------------------------------------------------------------
struct Topology {
  int world = 0;
  int kind = 0;  // 0 ring, 1 tree, 2 graph
  int branching = 2;
  std::vector<std::vector<int>> adj;
};

void topo_link(Topology& t, int a, int b) {
  if (a == b) return;
  auto add = [&](int u, int v) {
    auto& l = t.adj[u];
    if (std::find(l.begin(), l.end(), v) == l.end()) l.push_back(v);
  };
  add(a, b);
  add(b, a);
}

// breadth-first search: shortest hop path, ties resolved towards lower rank ids
int topo_route(const Topology& t, int src, int dst, int* out, int cap) {
  if (src < 0 || dst < 0 || src >= t.world || dst >= t.world) return -1;
  std::vector<int> prev(t.world, -2);
  std::deque<int> q{src};
  prev[src] = -1;
  while (!q.empty()) {
    int u = q.front();
    q.pop_front();
    if (u == dst) break;
    std::vector<int> nb = t.adj[u];
    std::sort(nb.begin(), nb.end());
    for (int v : nb)
      if (prev[v] == -2) {
        prev[v] = u;
        q.push_back(v);
      }
  }
  if (prev[dst] == -2) return -1;
  std::vector<int> path;
  for (int v = dst; v != -1; v = prev[v]) path.push_back(v);
  std::reverse(path.begin(), path.end());
  if ((int)path.size() > cap) return -(int)path.size();
  std::copy(path.begin(), path.end(), out);
  return (int)path.size();
}

// ---------------------------------------------------------------------------------------------------------------
// Framed TCP
// ---------------------------------------------------------------------------------------------------------------
int send_all(int fd, const void* p, size_t n) {
  const char* c = (const char*)p;
  while (n) {
    ssize_t k = ::send(fd, c, n, MSG_NOSIGNAL);
    if (k <= 0) return -1;
    c += k;
    n -= (size_t)k;
  }
  return 0;
}

int recv_all(int fd, void* p, size_t n) {
  char* c = (char*)p;
  while (n) {
    ssize_t k = ::recv(fd, c, n, 0);
    if (k <= 0) return -1;
    c += k;
    n -= (size_t)k;
  }
  return 0;
}

// frame = u32 type (LE) | u64 length (LE) | payload
int send_frame(int fd, uint32_t type, const void* p, uint64_t n) {
  char h[12];
  memcpy(h, &type, 4);
  memcpy(h + 4, &n, 8);
  if (send_all(fd, h, 12)) return -1;
  return n ? send_all(fd, p, n) : 0;
}

int recv_frame(int fd, uint32_t* type, std::vector<char>& buf, uint64_t max_len = (1ull << 32)) {
  char h[12];
  if (recv_all(fd, h, 12)) return -1;
  uint64_t n;
  memcpy(type, h, 4);
  memcpy(&n, h + 4, 8);
  if (n > max_len) return -2;
  buf.resize(n);
  return n ? recv_all(fd, buf.data(), n) : 0;
}

int tcp_listen(int port, int* bound_port) {
  int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return -1;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  a.sin_port = htons((uint16_t)port);
  if (::bind(fd, (sockaddr*)&a, sizeof a) || ::listen(fd, 64)) {
    ::close(fd);
    return -1;
  }
  socklen_t l = sizeof a;
  getsockname(fd, (sockaddr*)&a, &l);
  if (bound_port) *bound_port = ntohs(a.sin_port);
  return fd;
}

int tcp_connect(const char* host, int port, int timeout_ms) {
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    int fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) return -1;
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, host, &a.sin_addr) != 1) {
      ::close(fd);
      return -1;
    }
    if (::connect(fd, (sockaddr*)&a, sizeof a) == 0) {
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
      return fd;
    }
    ::close(fd);
    if (std::chrono::steady_clock::now() > deadline) return -1;
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
  }
}

void set_timeout(int fd, int ms) {
  timeval tv{ms / 1000, (ms % 1000) * 1000};
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
  setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof tv);
}

}  // namespace

// ----- topology C ABI ------------------------------------------------------------------------------------------
SX_EXPORT void* sx_topo_ring(int world) {
  if (world <= 0) return nullptr;
  auto* t = new Topology;
  t->world = world;
  t->kind = 0;
  t->adj.resize(world);
  for (int r = 0; r < world; ++r) topo_link(*t, r, (r + 1) % world);
  return t;
}

SX_EXPORT void* sx_topo_tree(int world, int branching) {
  if (world <= 0 || branching < 1) return nullptr;
  auto* t = new Topology;
  t->world = world;
  t->kind = 1;
  t->branching = branching;
  t->adj.resize(world);
  for (int r = 1; r < world; ++r) topo_link(*t, r, (r - 1) / branching);
  return t;
}

SX_EXPORT void* sx_topo_graph(int world, const int* adjacency) {
  if (world <= 0 || !adjacency) return nullptr;
  auto* t = new Topology;
  t->world = world;
  t->kind = 2;
  t->adj.resize(world);
  for (int i = 0; i < world; ++i)
    for (int j = 0; j < world; ++j)
      if (adjacency[i * world + j]) topo_link(*t, i, j);
  return t;
}

SX_EXPORT void sx_topo_destroy(void* h) { delete (Topology*)h; }

SX_EXPORT int sx_topo_next(void* h, int rank) {
  auto* t = (Topology*)h;
  return (t->kind == 0 && rank >= 0 && rank < t->world) ? (rank + 1) % t->world : -1;
}

SX_EXPORT int sx_topo_prev(void* h, int rank) {
  auto* t = (Topology*)h;
  return (t->kind == 0 && rank >= 0 && rank < t->world) ? (rank + t->world - 1) % t->world : -1;
}

SX_EXPORT int sx_topo_parent(void* h, int rank) {
  auto* t = (Topology*)h;
  return (t->kind == 1 && rank > 0 && rank < t->world) ? (rank - 1) / t->branching : -1;
}

SX_EXPORT int sx_topo_children(void* h, int rank, int* out, int cap) {
  auto* t = (Topology*)h;
  if (t->kind != 1 || rank < 0 || rank >= t->world) return -1;
  int n = 0;
  for (int c = rank * t->branching + 1; c <= rank * t->branching + t->branching && c < t->world; ++c)
    if (n < cap) out[n++] = c;
  return n;
}

SX_EXPORT int sx_topo_route(void* h, int src, int dst, int* out, int cap) { return topo_route(*(Topology*)h, src, dst, out, cap); }

// ----- framed socket C ABI -------------------------------------------------------------------------------------
SX_EXPORT int sx_sock_listen(int port, int* bound_port) { return tcp_listen(port, bound_port); }

SX_EXPORT int sx_sock_accept(int lfd, int timeout_ms) {
  pollfd p{lfd, POLLIN, 0};
  if (::poll(&p, 1, timeout_ms) <= 0) return -1;
  int fd = ::accept(lfd, nullptr, nullptr);
  if (fd >= 0) {
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
  }
  return fd;
}

SX_EXPORT int sx_sock_connect(const char* host, int port, int timeout_ms) { return tcp_connect(host, port, timeout_ms); }
SX_EXPORT void sx_sock_set_timeout(int fd, int ms) { set_timeout(fd, ms); }
SX_EXPORT void sx_sock_close(int fd) {
  if (fd >= 0) ::close(fd);
}
SX_EXPORT int sx_sock_send_message(int fd, const void* p, long long n) { return send_frame(fd, 1, p, (uint64_t)n); }

// Receives one message into `buf`; returns its length, -1 on a closed / timed-out socket, -(len) - 2 if `cap` is short
// (the message is consumed and dropped in that case).
SX_EXPORT long long sx_sock_recv_message(int fd, void* buf, long long cap) {
  uint32_t ty;
  std::vector<char> v;
  if (recv_frame(fd, &ty, v)) return -1;
  if ((long long)v.size() > cap) return -(long long)v.size() - 2;
  memcpy(buf, v.data(), v.size());
  return (long long)v.size();
}

// tensor on the wire: u32 dtype code | u32 ndim | i64 dims[ndim] | raw bytes
SX_EXPORT int sx_sock_send_tensor(int fd, const void* data, int dtype, int ndim, const long long* dims, long long nbytes) {
  std::vector<char> head(8 + 8 * (size_t)ndim);
  uint32_t d = (uint32_t)dtype, nd = (uint32_t)ndim;
  memcpy(head.data(), &d, 4);
  memcpy(head.data() + 4, &nd, 4);
  memcpy(head.data() + 8, dims, 8 * (size_t)ndim);
  if (send_frame(fd, 2, head.data(), head.size())) return -1;
  return send_frame(fd, 3, data, (uint64_t)nbytes);
}

SX_EXPORT long long sx_sock_recv_tensor(int fd, void* data, long long cap, int* dtype, int* ndim, long long* dims, int max_dims) {
  uint32_t ty;
  std::vector<char> head, body;
  if (recv_frame(fd, &ty, head) || ty != 2 || head.size() < 8) return -1;
  uint32_t d, nd;
  memcpy(&d, head.data(), 4);
  memcpy(&nd, head.data() + 4, 4);
  if ((int)nd > max_dims || head.size() != 8 + 8 * (size_t)nd) return -1;
  memcpy(dims, head.data() + 8, 8 * (size_t)nd);
  *dtype = (int)d;
  *ndim = (int)nd;
  if (recv_frame(fd, &ty, body) || ty != 3) return -1;
  if ((long long)body.size() > cap) return -(long long)body.size() - 2;
  memcpy(data, body.data(), body.size());
  return (long long)body.size();
}

// ---------------------------------------------------------------------------------------------------------------
// Coordinator: one server, `world` clients. Verbs: register (token checked), rank / world, barrier, all-gather of
// equal-size blobs, relayed point-to-point blobs. One thread per connection; collective verbs block in the server
// until every rank has arrived (generation counted, so they can be repeated).
// ---------------------------------------------------------------------------------------------------------------
namespace {

enum : uint32_t { V_REGISTER = 10, V_BARRIER, V_ALLGATHER, V_SEND, V_RECV, V_INFO, V_OK = 100, V_ERR = 101 };

struct Coordinator {
  int lfd = -1, port = 0, world = 0;
  std::string token;
  std::atomic<bool> stop{false};
  std::thread acceptor;
  std::vector<std::thread> workers;
  std::mutex mu;
  std::condition_variable cv;
  int next_rank = 0;
  std::map<std::string, int> names;  // node name -> rank (re-registration keeps the rank)
  int bar_count = 0;
  long long bar_gen = 0;
  int ag_count = 0;
  long long ag_gen = 0;
  std::vector<std::vector<char>> ag_slots, ag_result;
  std::map<std::pair<int, int>, std::deque<std::vector<char>>> mail;  // (src, dst) -> queue
  std::vector<int> fds;

  void serve(int fd) {
    int rank = -1;
    std::vector<char> buf;
    uint32_t ty;
    while (!stop && recv_frame(fd, &ty, buf, 1ull << 30) == 0) {
      if (ty == V_REGISTER) {
        // payload: u32 token_len | token | name
        uint32_t tl = 0;
        if (buf.size() >= 4) memcpy(&tl, buf.data(), 4);
        if (buf.size() < 4 + (size_t)tl) { send_frame(fd, V_ERR, "malformed", 9); continue; }
        std::string tok(buf.data() + 4, tl), name(buf.data() + 4 + tl, buf.size() - 4 - tl);
        std::unique_lock<std::mutex> lk(mu);
        if (tok != token) { lk.unlock(); send_frame(fd, V_ERR, "unauthenticated", 15); continue; }
        auto it = names.find(name);
        if (it != names.end()) rank = it->second;
        else if (next_rank < world) { rank = next_rank++; names[name] = rank; }
        else { lk.unlock(); send_frame(fd, V_ERR, "world full", 10); continue; }
        cv.notify_all();
        lk.unlock();
        int32_t out[2] = {rank, world};
        send_frame(fd, V_OK, out, 8);
        continue;
      }
      if (rank < 0) { send_frame(fd, V_ERR, "not registered", 14); continue; }
      if (ty == V_INFO) {
        std::unique_lock<std::mutex> lk(mu);
        int32_t out[3] = {rank, world, next_rank};
        lk.unlock();
        send_frame(fd, V_OK, out, 12);
      } else if (ty == V_BARRIER) {
        std::unique_lock<std::mutex> lk(mu);
        long long g = bar_gen;
        if (++bar_count == world) { bar_count = 0; ++bar_gen; cv.notify_all(); }
        else cv.wait(lk, [&] { return bar_gen != g || stop.load(); });
        lk.unlock();
        send_frame(fd, stop ? V_ERR : V_OK, nullptr, 0);
      } else if (ty == V_ALLGATHER) {
        std::unique_lock<std::mutex> lk(mu);
        long long g = ag_gen;
        if ((int)ag_slots.size() != world) ag_slots.assign(world, {});
        ag_slots[rank] = buf;
        if (++ag_count == world) { ag_result = ag_slots; ag_count = 0; ++ag_gen; cv.notify_all(); }
        else cv.wait(lk, [&] { return ag_gen != g || stop.load(); });
        std::vector<char> out;
        for (auto& s : ag_result) out.insert(out.end(), s.begin(), s.end());
        lk.unlock();
        send_frame(fd, stop ? V_ERR : V_OK, out.data(), out.size());
      } else if (ty == V_SEND) {
        int32_t dst = -1;
        if (buf.size() >= 4) memcpy(&dst, buf.data(), 4);
        if (dst < 0 || dst >= world) { send_frame(fd, V_ERR, "bad rank", 8); continue; }
        {
          std::lock_guard<std::mutex> lk(mu);
          mail[{rank, dst}].emplace_back(buf.begin() + 4, buf.end());
          cv.notify_all();
        }
        send_frame(fd, V_OK, nullptr, 0);
      } else if (ty == V_RECV) {
        int32_t src = -1, tmo = 5000;
        if (buf.size() >= 8) { memcpy(&src, buf.data(), 4); memcpy(&tmo, buf.data() + 4, 4); }
        std::unique_lock<std::mutex> lk(mu);
        auto key = std::make_pair((int)src, rank);
        bool ok = cv.wait_for(lk, std::chrono::milliseconds(tmo), [&] { return !mail[key].empty() || stop.load(); });
        if (!ok || mail[key].empty()) { lk.unlock(); send_frame(fd, V_ERR, "timeout", 7); continue; }
        std::vector<char> m = std::move(mail[key].front());
        mail[key].pop_front();
        lk.unlock();
        send_frame(fd, V_OK, m.data(), m.size());
      } else {
        send_frame(fd, V_ERR, "unknown verb", 12);
      }
    }
    ::close(fd);
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
      fds.push_back(fd);
      workers.emplace_back([this, fd] { serve(fd); });
    }
  }
};

struct CoordClient {
  int fd = -1, rank = -1, world = 0;
  std::string err;
};

int coord_call(CoordClient* c, uint32_t verb, const void* p, uint64_t n, std::vector<char>& reply) {
  uint32_t ty;
  if (send_frame(c->fd, verb, p, n) || recv_frame(c->fd, &ty, reply)) { c->err = "connection lost"; return -1; }
  if (ty != V_OK) { c->err.assign(reply.begin(), reply.end()); return -2; }
  return 0;
}

}  // namespace

SX_EXPORT void* sx_coord_server_start(int port, int world, const char* token) {
  auto* s = new Coordinator;
  s->world = world;
  s->token = token ? token : "";
  s->lfd = tcp_listen(port, &s->port);
  if (s->lfd < 0) { delete s; return nullptr; }
  s->acceptor = std::thread([s] { s->accept_loop(); });
  return s;
}

SX_EXPORT int sx_coord_server_port(void* h) { return ((Coordinator*)h)->port; }

SX_EXPORT void sx_coord_server_stop(void* h) {
  auto* s = (Coordinator*)h;
  s->stop = true;
  {
    std::lock_guard<std::mutex> lk(s->mu);
    s->cv.notify_all();
    for (int fd : s->fds) ::shutdown(fd, SHUT_RDWR);
  }
  if (s->acceptor.joinable()) s->acceptor.join();
  for (auto& w : s->workers)
    if (w.joinable()) w.join();
  ::close(s->lfd);
  delete s;
}

SX_EXPORT void* sx_coord_connect(const char* host, int port, int timeout_ms) {
  int fd = tcp_connect(host, port, timeout_ms);
  if (fd < 0) return nullptr;
  auto* c = new CoordClient;
  c->fd = fd;
  return c;
}

SX_EXPORT void sx_coord_close(void* h) {
  auto* c = (CoordClient*)h;
  if (c->fd >= 0) ::close(c->fd);
  delete c;
}

SX_EXPORT const char* sx_coord_error(void* h) { return ((CoordClient*)h)->err.c_str(); }

// returns the assigned rank (>= 0), -1 on a lost connection, -2 when the server refused (see sx_coord_error)
SX_EXPORT int sx_coord_register(void* h, const char* token, const char* name) {
  auto* c = (CoordClient*)h;
  std::string t = token ? token : "", n = name ? name : "";
  std::vector<char> msg(4 + t.size() + n.size());
  uint32_t tl = (uint32_t)t.size();
  memcpy(msg.data(), &tl, 4);
  memcpy(msg.data() + 4, t.data(), t.size());
  memcpy(msg.data() + 4 + t.size(), n.data(), n.size());
  std::vector<char> r;
  int rc = coord_call(c, V_REGISTER, msg.data(), msg.size(), r);
  if (rc) return rc;
  int32_t out[2];
  memcpy(out, r.data(), 8);
  c->rank = out[0];
  c->world = out[1];
  return c->rank;
}

SX_EXPORT int sx_coord_world(void* h) { return ((CoordClient*)h)->world; }
SX_EXPORT int sx_coord_rank(void* h) { return ((CoordClient*)h)->rank; }

SX_EXPORT int sx_coord_barrier(void* h) {
  std::vector<char> r;
  return coord_call((CoordClient*)h, V_BARRIER, nullptr, 0, r);
}

// `recv` must hold world * nbytes
SX_EXPORT int sx_coord_all_gather(void* h, const void* send, long long nbytes, void* recv) {
  auto* c = (CoordClient*)h;
  std::vector<char> r;
  int rc = coord_call(c, V_ALLGATHER, send, (uint64_t)nbytes, r);
  if (rc) return rc;
  if ((long long)r.size() != nbytes * c->world) { c->err = "ranks sent different sizes"; return -3; }
  memcpy(recv, r.data(), r.size());
  return 0;
}

SX_EXPORT int sx_coord_send(void* h, int dst, const void* p, long long nbytes) {
  std::vector<char> msg(4 + (size_t)nbytes), r;
  int32_t d = dst;
  memcpy(msg.data(), &d, 4);
  memcpy(msg.data() + 4, p, (size_t)nbytes);
  return coord_call((CoordClient*)h, V_SEND, msg.data(), msg.size(), r);
}

SX_EXPORT long long sx_coord_recv(void* h, int src, void* p, long long cap, int timeout_ms) {
  int32_t q[2] = {src, timeout_ms};
  std::vector<char> r;
  int rc = coord_call((CoordClient*)h, V_RECV, q, 8, r);
  if (rc) return rc;
  if ((long long)r.size() > cap) return -(long long)r.size() - 2;
  memcpy(p, r.data(), r.size());
  return (long long)r.size();
}

// ---------------------------------------------------------------------------------------------------------------
// Raft. Nodes are pure state machines (no threads, no sockets): time advances through tick(), messages arrive through
// handle(). RaftCluster wires N of them through an in-memory network whose links can be cut, which is also how the
// tests inject failures.
// ---------------------------------------------------------------------------------------------------------------
namespace {

struct RaftEntry { int term; std::string data; };

struct RaftMsg {
  int kind;  // 0 RequestVote, 1 VoteReply, 2 AppendEntries, 3 AppendReply
  int from, to, term;
  int last_index = 0, last_term = 0;      // RequestVote
  bool granted = false;                   // VoteReply
  int prev_index = 0, prev_term = 0, leader_commit = 0;  // AppendEntries
  std::vector<RaftEntry> entries;
  bool success = false; int match = 0;    // AppendReply
};

struct RaftNode {
  enum { FOLLOWER, CANDIDATE, LEADER };
  int id = 0, n = 0, role = FOLLOWER, term = 0, voted_for = -1, leader = -1;
  int commit = 0, applied = 0, votes = 0;
  std::vector<RaftEntry> log;  // log[0] is entry index 1
  std::vector<int> next_idx, match_idx;
  int election_ms = 150, heartbeat_ms = 50, elapsed = 0, timeout = 0;
  uint64_t rng = 1;
  std::vector<RaftMsg>* out = nullptr;

  int rnd() { rng = rng * 6364136223846793005ull + 1442695040888963407ull; return (int)(rng >> 33); }
  void reset_timer() { elapsed = 0; timeout = election_ms + rnd() % election_ms; }
  int last_index() const { return (int)log.size(); }
  int term_at(int i) const { return i == 0 ? 0 : log[i - 1].term; }

  void become_follower(int t) { role = FOLLOWER; term = t; voted_for = -1; reset_timer(); }

  void start_election() {
    role = CANDIDATE; ++term; voted_for = id; votes = 1; leader = -1; reset_timer();
    if (n == 1) { become_leader(); return; }
    for (int p = 0; p < n; ++p) if (p != id) {
      RaftMsg m{0, id, p, term}; m.last_index = last_index(); m.last_term = term_at(last_index());
      out->push_back(m);
    }
  }

  void become_leader() {
    role = LEADER; leader = id;
    next_idx.assign(n, last_index() + 1); match_idx.assign(n, 0); match_idx[id] = last_index();
    broadcast();
  }

  void send_append(int p) {
    RaftMsg m{2, id, p, term};
    m.prev_index = next_idx[p] - 1; m.prev_term = term_at(m.prev_index); m.leader_commit = commit;
    for (int i = next_idx[p]; i <= last_index(); ++i) m.entries.push_back(log[i - 1]);
    out->push_back(m);
  }

  void broadcast() { elapsed = 0; for (int p = 0; p < n; ++p) if (p != id) send_append(p); }

  void advance_commit() {
    for (int idx = last_index(); idx > commit; --idx) {
      if (term_at(idx) != term) break;  // only entries of the current term commit by counting
      int cnt = 0;
      for (int p = 0; p < n; ++p) if (match_idx[p] >= idx) ++cnt;
      if (cnt * 2 > n) { commit = idx; break; }
    }
    applied = commit;
  }

  void tick(int ms) {
    elapsed += ms;
    if (role == LEADER) { if (elapsed >= heartbeat_ms) broadcast(); }
    else if (elapsed >= timeout) start_election();
  }

  int propose(const char* d, size_t len) {
    if (role != LEADER) return -1;
    log.push_back({term, std::string(d, len)});
    match_idx[id] = last_index();
    if (n == 1) advance_commit(); else broadcast();
    return last_index();
  }

  void handle(const RaftMsg& m) {
    if (m.term > term) become_follower(m.term);
    switch (m.kind) {
      case 0: {
        bool up_to_date = m.last_term > term_at(last_index()) ||
                          (m.last_term == term_at(last_index()) && m.last_index >= last_index());
        bool grant = m.term == term && (voted_for == -1 || voted_for == m.from) && up_to_date;
        if (grant) { voted_for = m.from; reset_timer(); }
        RaftMsg r{1, id, m.from, term}; r.granted = grant; out->push_back(r);
        break;
      }
      case 1:
        if (role == CANDIDATE && m.term == term && m.granted && ++votes * 2 > n) become_leader();
        break;
      case 2: {
        RaftMsg r{3, id, m.from, term};
        if (m.term < term) { r.success = false; out->push_back(r); break; }
        role = FOLLOWER; leader = m.from; reset_timer();
        if (m.prev_index > last_index() || term_at(m.prev_index) != m.prev_term) {
          r.success = false; r.match = std::min(last_index(), m.prev_index - 1); out->push_back(r); break;
        }
        int idx = m.prev_index;
        for (auto& e : m.entries) {
          ++idx;
          if (idx <= last_index() && term_at(idx) != e.term) log.resize(idx - 1);
          if (idx > last_index()) log.push_back(e);
        }
        if (m.leader_commit > commit) { commit = std::min(m.leader_commit, idx); applied = commit; }
        r.success = true; r.match = idx; out->push_back(r);
        break;
      }
      case 3:
        if (role != LEADER || m.term != term) break;
        if (m.success) { match_idx[m.from] = std::max(match_idx[m.from], m.match); next_idx[m.from] = match_idx[m.from] + 1; advance_commit(); }
        else { next_idx[m.from] = std::max(1, std::min(next_idx[m.from] - 1, m.match + 1)); send_append(m.from); }
        break;
    }
  }
};

struct RaftCluster {
  std::vector<RaftNode> nodes;
  std::vector<RaftMsg> wire;
  std::vector<char> connected;

  void step(int ms) {
    for (size_t i = 0; i < nodes.size(); ++i) if (connected[i]) nodes[i].tick(ms);
    // deliver until quiet (bounded: replies can trigger at most a few rounds per step)
    for (int round = 0; round < 16 && !wire.empty(); ++round) {
      std::vector<RaftMsg> batch; batch.swap(wire);
      for (auto& m : batch) if (connected[m.from] && connected[m.to]) nodes[m.to].handle(m);
    }
  }
};

}  // namespace

SX_EXPORT void* sx_raft_cluster_create(int n, int election_ms, int heartbeat_ms, unsigned long long seed) {
  if (n < 1) return nullptr;
  auto* c = new RaftCluster;
  c->nodes.resize(n); c->connected.assign(n, 1);
  for (int i = 0; i < n; ++i) {
    auto& nd = c->nodes[i];
    nd.id = i; nd.n = n; nd.election_ms = election_ms; nd.heartbeat_ms = heartbeat_ms; nd.rng = seed * 977 + i * 7919 + 1;
    nd.out = &c->wire; nd.reset_timer();
  }
  return c;
}
SX_EXPORT void sx_raft_cluster_destroy(void* h) { delete (RaftCluster*)h; }
SX_EXPORT void sx_raft_cluster_step(void* h, int ms) { ((RaftCluster*)h)->step(ms); }
SX_EXPORT void sx_raft_cluster_set_connected(void* h, int node, int on) { ((RaftCluster*)h)->connected[node] = (char)on; }

// the connected leader with the highest term, or -1
SX_EXPORT int sx_raft_cluster_leader(void* h) {
  auto* c = (RaftCluster*)h; int best = -1;
  for (auto& nd : c->nodes)
    if (c->connected[nd.id] && nd.role == RaftNode::LEADER && (best < 0 || nd.term > c->nodes[best].term)) best = nd.id;
  return best;
}
SX_EXPORT int sx_raft_cluster_propose(void* h, int node, const void* data, long long len) {
  auto* c = (RaftCluster*)h;
  if (!c->connected[node]) return -1;
  int idx = c->nodes[node].propose((const char*)data, (size_t)len);
  c->step(0);
  return idx;
}
// out = {term, commit_index, last_applied, role, log_length, known_leader}
SX_EXPORT void sx_raft_cluster_state(void* h, int node, int* out) {
  auto& nd = ((RaftCluster*)h)->nodes[node];
  out[0] = nd.term; out[1] = nd.commit; out[2] = nd.applied; out[3] = nd.role; out[4] = nd.last_index(); out[5] = nd.leader;
}
SX_EXPORT long long sx_raft_cluster_entry(void* h, int node, int index, void* buf, long long cap) {
  auto& nd = ((RaftCluster*)h)->nodes[node];
  if (index < 1 || index > nd.last_index()) return -1;
  auto& d = nd.log[index - 1].data;
  if ((long long)d.size() > cap) return -(long long)d.size() - 2;
  memcpy(buf, d.data(), d.size());
  return (long long)d.size();
}

// ---------------------------------------------------------------------------------------------------------------
// Health check: a node is healthy while its last report is younger than `timeout_ms` and its failure streak is below
// `max_failures`.
// ---------------------------------------------------------------------------------------------------------------
namespace {
struct Health {
  struct Rec { double last_ms = -1; int fails = 0; double latency_ms = 0; };
  std::map<int, Rec> recs; double timeout_ms; int max_failures; std::mutex mu;
};
}  // namespace
SX_EXPORT void* sx_health_create(double timeout_ms, int max_failures) { auto* h = new Health; h->timeout_ms = timeout_ms; h->max_failures = max_failures; return h; }
SX_EXPORT void sx_health_destroy(void* h) { delete (Health*)h; }
SX_EXPORT void sx_health_report(void* hh, int node, double now_ms, int ok, double latency_ms) {
  auto* h = (Health*)hh; std::lock_guard<std::mutex> lk(h->mu);
  auto& r = h->recs[node];
  if (ok) { r.last_ms = now_ms; r.fails = 0; r.latency_ms = r.latency_ms == 0 ? latency_ms : 0.8 * r.latency_ms + 0.2 * latency_ms; }
  else ++r.fails;
}
// 1 healthy, 0 unhealthy, -1 never seen
SX_EXPORT int sx_health_status(void* hh, int node, double now_ms) {
  auto* h = (Health*)hh; std::lock_guard<std::mutex> lk(h->mu);
  auto it = h->recs.find(node);
  if (it == h->recs.end() || it->second.last_ms < 0) return it == h->recs.end() ? -1 : 0;
  return (now_ms - it->second.last_ms <= h->timeout_ms && it->second.fails < h->max_failures) ? 1 : 0;
}
SX_EXPORT double sx_health_latency(void* hh, int node) {
  auto* h = (Health*)hh; std::lock_guard<std::mutex> lk(h->mu);
  auto it = h->recs.find(node); return it == h->recs.end() ? -1.0 : it->second.latency_ms;
}

// ---------------------------------------------------------------------------------------------------------------
// WebSocket (RFC 6455): accept-key derivation and frame encode / decode. MQTT 3.1.1: CONNECT / PUBLISH / SUBSCRIBE
// packets, remaining-length varint, topic-filter matching. Service directory: name -> endpoint records with TTL.
// ---------------------------------------------------------------------------------------------------------------
namespace {

void sha1(const uint8_t* msg, size_t len, uint8_t out[20]) {
  uint32_t h[5] = {0x67452301u, 0xEFCDAB89u, 0x98BADCFEu, 0x10325476u, 0xC3D2E1F0u};
  std::vector<uint8_t> m(msg, msg + len);
  m.push_back(0x80);
  while (m.size() % 64 != 56) m.push_back(0);
  uint64_t bits = (uint64_t)len * 8;
  for (int i = 7; i >= 0; --i) m.push_back((uint8_t)(bits >> (8 * i)));
  auto rol = [](uint32_t x, int s) { return (x << s) | (x >> (32 - s)); };
  for (size_t off = 0; off < m.size(); off += 64) {
    uint32_t w[80];
    for (int i = 0; i < 16; ++i) w[i] = (uint32_t)m[off + 4 * i] << 24 | (uint32_t)m[off + 4 * i + 1] << 16 | (uint32_t)m[off + 4 * i + 2] << 8 | m[off + 4 * i + 3];
    for (int i = 16; i < 80; ++i) w[i] = rol(w[i - 3] ^ w[i - 8] ^ w[i - 14] ^ w[i - 16], 1);
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4];
    for (int i = 0; i < 80; ++i) {
      uint32_t f, k;
      if (i < 20) { f = (b & c) | (~b & d); k = 0x5A827999u; }
      else if (i < 40) { f = b ^ c ^ d; k = 0x6ED9EBA1u; }
      else if (i < 60) { f = (b & c) | (b & d) | (c & d); k = 0x8F1BBCDCu; }
      else { f = b ^ c ^ d; k = 0xCA62C1D6u; }
      uint32_t t = rol(a, 5) + f + e + k + w[i];
      e = d; d = c; c = rol(b, 30); b = a; a = t;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e;
  }
  for (int i = 0; i < 5; ++i) for (int j = 0; j < 4; ++j) out[4 * i + j] = (uint8_t)(h[i] >> (24 - 8 * j));
}

std::string base64(const uint8_t* p, size_t n) {
  static const char* T = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";
  std::string o;
  for (size_t i = 0; i < n; i += 3) {
    uint32_t v = p[i] << 16 | (i + 1 < n ? p[i + 1] << 8 : 0) | (i + 2 < n ? p[i + 2] : 0);
    o += T[v >> 18 & 63]; o += T[v >> 12 & 63];
    o += i + 1 < n ? T[v >> 6 & 63] : '='; o += i + 2 < n ? T[v & 63] : '=';
  }
  return o;
}

}  // namespace

SX_EXPORT void sx_sha1(const void* msg, long long len, void* out20) { sha1((const uint8_t*)msg, (size_t)len, (uint8_t*)out20); }

// Sec-WebSocket-Accept for a client's Sec-WebSocket-Key; `out` needs 29 bytes
SX_EXPORT void sx_ws_accept_key(const char* client_key, char* out) {
  std::string s = std::string(client_key) + "258EAFA5-E914-47DA-95CA-C5AB0DC85B11";
  uint8_t d[20]; sha1((const uint8_t*)s.data(), s.size(), d);
  std::string b = base64(d, 20); memcpy(out, b.c_str(), b.size() + 1);
}

// Encodes one frame (FIN set). mask_key == 0 sends unmasked (server side). Returns bytes written or -needed.
SX_EXPORT long long sx_ws_encode(int opcode, const void* payload, long long n, unsigned mask_key, void* out, long long cap) {
  long long need = 2 + (n < 126 ? 0 : n < 65536 ? 2 : 8) + (mask_key ? 4 : 0) + n;
  if (need > cap) return -need;
  uint8_t* o = (uint8_t*)out; size_t k = 0;
  o[k++] = 0x80 | (opcode & 0xF);
  uint8_t mb = mask_key ? 0x80 : 0;
  if (n < 126) o[k++] = mb | (uint8_t)n;
  else if (n < 65536) { o[k++] = mb | 126; o[k++] = (uint8_t)(n >> 8); o[k++] = (uint8_t)n; }
  else { o[k++] = mb | 127; for (int i = 7; i >= 0; --i) o[k++] = (uint8_t)((uint64_t)n >> (8 * i)); }
  uint8_t mk[4] = {(uint8_t)(mask_key >> 24), (uint8_t)(mask_key >> 16), (uint8_t)(mask_key >> 8), (uint8_t)mask_key};
  if (mask_key) for (int i = 0; i < 4; ++i) o[k++] = mk[i];
  const uint8_t* p = (const uint8_t*)payload;
  for (long long i = 0; i < n; ++i) o[k++] = mask_key ? p[i] ^ mk[i & 3] : p[i];
  return (long long)k;
}

// Decodes one frame from `in`. Returns bytes consumed (0 = need more data, <0 = malformed); payload is unmasked into out.
SX_EXPORT long long sx_ws_decode(const void* in, long long n, int* opcode, int* fin, void* out, long long cap, long long* payload_len) {
  const uint8_t* p = (const uint8_t*)in;
  if (n < 2) return 0;
  *fin = p[0] >> 7; *opcode = p[0] & 0xF;
  bool masked = p[1] & 0x80; uint64_t len = p[1] & 0x7F; size_t k = 2;
  if (len == 126) { if (n < 4) return 0; len = (uint64_t)p[2] << 8 | p[3]; k = 4; }
  else if (len == 127) { if (n < 10) return 0; len = 0; for (int i = 0; i < 8; ++i) len = len << 8 | p[2 + i]; k = 10; }
  uint8_t mk[4] = {0, 0, 0, 0};
  if (masked) { if ((size_t)n < k + 4) return 0; memcpy(mk, p + k, 4); k += 4; }
  if ((uint64_t)n < k + len) return 0;
  if ((long long)len > cap) return -1;
  uint8_t* o = (uint8_t*)out;
  for (uint64_t i = 0; i < len; ++i) o[i] = masked ? p[k + i] ^ mk[i & 3] : p[k + i];
  *payload_len = (long long)len;
  return (long long)(k + len);
}

namespace {
void mqtt_varint(std::vector<uint8_t>& o, uint32_t v) { do { uint8_t b = v % 128; v /= 128; if (v) b |= 0x80; o.push_back(b); } while (v); }
void mqtt_str(std::vector<uint8_t>& o, const char* s) { size_t n = strlen(s); o.push_back((uint8_t)(n >> 8)); o.push_back((uint8_t)n); o.insert(o.end(), s, s + n); }
long long mqtt_emit(uint8_t head, const std::vector<uint8_t>& body, void* out, long long cap) {
  std::vector<uint8_t> pkt{head}; mqtt_varint(pkt, (uint32_t)body.size()); pkt.insert(pkt.end(), body.begin(), body.end());
  if ((long long)pkt.size() > cap) return -(long long)pkt.size();
  memcpy(out, pkt.data(), pkt.size()); return (long long)pkt.size();
}
}  // namespace

SX_EXPORT long long sx_mqtt_connect(const char* client_id, int keepalive_s, int clean, void* out, long long cap) {
  std::vector<uint8_t> b; mqtt_str(b, "MQTT"); b.push_back(4); b.push_back(clean ? 2 : 0);
  b.push_back((uint8_t)(keepalive_s >> 8)); b.push_back((uint8_t)keepalive_s); mqtt_str(b, client_id);
  return mqtt_emit(0x10, b, out, cap);
}
SX_EXPORT long long sx_mqtt_publish(const char* topic, const void* payload, long long n, int qos, int retain, int packet_id, void* out, long long cap) {
  std::vector<uint8_t> b; mqtt_str(b, topic);
  if (qos > 0) { b.push_back((uint8_t)(packet_id >> 8)); b.push_back((uint8_t)packet_id); }
  b.insert(b.end(), (const uint8_t*)payload, (const uint8_t*)payload + n);
  return mqtt_emit((uint8_t)(0x30 | (qos << 1) | (retain ? 1 : 0)), b, out, cap);
}
SX_EXPORT long long sx_mqtt_subscribe(const char* filter, int qos, int packet_id, void* out, long long cap) {
  std::vector<uint8_t> b{(uint8_t)(packet_id >> 8), (uint8_t)packet_id}; mqtt_str(b, filter); b.push_back((uint8_t)qos);
  return mqtt_emit(0x82, b, out, cap);
}
// Parses the fixed header: returns header length (0 = need more, -1 = malformed), fills type / flags / remaining length
SX_EXPORT int sx_mqtt_parse_header(const void* in, long long n, int* type, int* flags, long long* remaining) {
  const uint8_t* p = (const uint8_t*)in;
  if (n < 2) return 0;
  *type = p[0] >> 4; *flags = p[0] & 0xF;
  uint32_t v = 0, mult = 1; int k = 1;
  for (;; ++k) { if (k >= n) return 0; if (k > 4) return -1; v += (p[k] & 0x7F) * mult; mult *= 128; if (!(p[k] & 0x80)) break; }
  *remaining = v; return k + 1;
}
// Decodes a PUBLISH body (after the fixed header). Returns payload offset within body, or -1.
SX_EXPORT long long sx_mqtt_parse_publish(const void* body, long long n, int flags, char* topic, int topic_cap, int* packet_id) {
  const uint8_t* p = (const uint8_t*)body;
  if (n < 2) return -1;
  int tl = p[0] << 8 | p[1];
  if (2 + tl > n || tl + 1 > topic_cap) return -1;
  memcpy(topic, p + 2, tl); topic[tl] = 0;
  long long k = 2 + tl; *packet_id = 0;
  if ((flags >> 1) & 3) { if (k + 2 > n) return -1; *packet_id = p[k] << 8 | p[k + 1]; k += 2; }
  return k;
}
// MQTT topic filter match with + (one level) and # (rest); topics starting with $ do not match wildcard-first filters
SX_EXPORT int sx_mqtt_topic_match(const char* filter, const char* topic) {
  if (topic[0] == '$' && (filter[0] == '+' || filter[0] == '#')) return 0;
  auto split = [](const char* s) { std::vector<std::string> v(1); for (; *s; ++s) { if (*s == '/') v.emplace_back(); else v.back() += *s; } return v; };
  std::vector<std::string> f = split(filter), t = split(topic);
  for (size_t i = 0; i < f.size(); ++i) {
    if (f[i] == "#") return i + 1 == f.size();  // also matches the parent level: "a/#" matches "a"
    if (i >= t.size()) return 0;
    if (f[i] != "+" && f[i] != t[i]) return 0;
  }
  return f.size() == t.size();
}

namespace {
struct ServiceDir {
  struct Rec { std::string type, host, txt; int port; double expires_ms; };
  std::map<std::string, Rec> recs; std::mutex mu;
};
}  // namespace
SX_EXPORT void* sx_sd_create() { return new ServiceDir; }
SX_EXPORT void sx_sd_destroy(void* h) { delete (ServiceDir*)h; }
SX_EXPORT void sx_sd_register(void* hh, const char* name, const char* type, const char* host, int port, const char* txt, double now_ms, double ttl_ms) {
  auto* h = (ServiceDir*)hh; std::lock_guard<std::mutex> lk(h->mu);
  h->recs[name] = {type, host, txt ? txt : "", port, now_ms + ttl_ms};
}
SX_EXPORT int sx_sd_unregister(void* hh, const char* name) { auto* h = (ServiceDir*)hh; std::lock_guard<std::mutex> lk(h->mu); return (int)h->recs.erase(name); }
// Writes "name\thost\tport\ttxt\n" lines for live records of `type`; returns the record count
SX_EXPORT int sx_sd_browse(void* hh, const char* type, double now_ms, char* out, int cap) {
  auto* h = (ServiceDir*)hh; std::lock_guard<std::mutex> lk(h->mu);
  std::string s; int n = 0;
  for (auto it = h->recs.begin(); it != h->recs.end();) {
    if (it->second.expires_ms < now_ms) { it = h->recs.erase(it); continue; }
    if (it->second.type == type) { s += it->first + "\t" + it->second.host + "\t" + std::to_string(it->second.port) + "\t" + it->second.txt + "\n"; ++n; }
    ++it;
  }
  if ((int)s.size() + 1 > cap) return -(int)s.size() - 1;
  memcpy(out, s.c_str(), s.size() + 1); return n;
}
