// Host-side distributed runtime: point-to-point backends (TCP star / full mesh, in-process simulated fabric,
// sub-group views) and the collectives layered on their byte-level send/recv, with per-receive timeouts, typed
// error codes and host-side fault injection for failure-detection tests.
//
// Capability parity (behaviour, not code): Backend trait + TcpBackend + SimulatedBackend + SubBackend
// (ferrotorch-distributed/src/backend.rs:29-753: rank 0 listens, peers announce their rank as u64-LE, 8-byte LE
// length-prefixed frames, read-timeout based recv_timeout, gather/scatter barrier), star collectives with
// Sum/Mean in fixed rank order (collective.rs:64-682), ring all-reduce / binomial-tree broadcast / ring barrier
// (gloo_native/collectives.rs:85-300), typed errors (error.rs:8-52).
#include <cstdlib>
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/uio.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#define FT_API extern "C" __attribute__((visibility("default")))

namespace ft {

enum Err : int {
  OK = 0, E_INVALID_WORLD = 1, E_INVALID_RANK = 2, E_SELF_SEND = 3, E_SIZE_MISMATCH = 4, E_IO = 5, E_LOCK = 6,
  E_CHANNEL_CLOSED = 7, E_UNSUPPORTED = 8, E_TIMEOUT = 9, E_NO_CONNECTION = 10, E_BACKEND_UNAVAILABLE = 11, E_ARG = 12,
};

enum Fault : int { F_NONE = 0, F_DROP_NEXT_SEND = 1, F_DELAY_SEND_MS = 2, F_CORRUPT_LENGTH = 3, F_CLOSE = 4 };

using Clock = std::chrono::steady_clock;

struct Backend {
  virtual ~Backend() = default;
  virtual int rank() const = 0;
  virtual int world() const = 0;
  virtual int send(const void* data, size_t n, int dst) = 0;
  // receives exactly n bytes from src; timeout_ms < 0 waits forever
  virtual int recv(void* data, size_t n, int src, int64_t timeout_ms) = 0;
  virtual int barrier(int64_t timeout_ms) {
    // gather to 0 then release (the reference's star barrier, backend.rs:359-377)
    uint8_t b = 1;
    const int r = rank(), w = world();
    if (w == 1) return OK;
    if (r == 0) {
      for (int p = 1; p < w; p++) { int e = recv(&b, 1, p, timeout_ms); if (e) return e; }
      for (int p = 1; p < w; p++) { int e = send(&b, 1, p); if (e) return e; }
    } else {
      int e = send(&b, 1, 0); if (e) return e;
      e = recv(&b, 1, 0, timeout_ms); if (e) return e;
    }
    return OK;
  }
  // host-side fault injection (tests only)
  std::atomic<int> fault{F_NONE};
  std::atomic<int64_t> fault_param{0};
};

// ------------------------------------------------------------------------------------------------------------
// TCP
// ------------------------------------------------------------------------------------------------------------
static int read_full(int fd, void* buf, size_t n, int64_t timeout_ms) {
  uint8_t* p = static_cast<uint8_t*>(buf);
  auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms < 0 ? 0 : timeout_ms);
  while (n > 0) {
    // data that is already in the socket buffer is taken without a poll; the poll (with what is left of the deadline) only runs when the
    // socket is empty
    ssize_t got = ::recv(fd, p, n, MSG_DONTWAIT);
    if (got > 0) { p += got; n -= (size_t)got; continue; }
    if (got == 0) return E_CHANNEL_CLOSED;
    if (errno == EINTR) continue;
    if (errno != EAGAIN && errno != EWOULDBLOCK) return E_IO;
    int wait_ms = -1;
    if (timeout_ms >= 0) {
      auto left = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - Clock::now()).count();
      if (left <= 0) return E_TIMEOUT;
      wait_ms = (int)std::min<int64_t>(left, 1 << 30);
    }
    pollfd pfd{fd, POLLIN, 0};
    int pr = ::poll(&pfd, 1, wait_ms);
    if (pr == 0) return E_TIMEOUT;
    if (pr < 0) { if (errno == EINTR) continue; return E_IO; }
  }
  return OK;
}

static int write_full(int fd, const void* buf, size_t n) {
  const uint8_t* p = static_cast<const uint8_t*>(buf);
  while (n > 0) {
    ssize_t put = ::send(fd, p, n, MSG_NOSIGNAL);
    if (put < 0) { if (errno == EINTR) continue; return (errno == EPIPE || errno == ECONNRESET) ? E_CHANNEL_CLOSED : E_IO; }
    p += put; n -= (size_t)put;
  }
  return OK;
}

static void put_u64le(uint8_t* b, uint64_t v) { for (int i = 0; i < 8; i++) b[i] = (uint8_t)(v >> (8 * i)); }
static uint64_t get_u64le(const uint8_t* b) { uint64_t v = 0; for (int i = 0; i < 8; i++) v |= (uint64_t)b[i] << (8 * i); return v; }

class TcpBackend : public Backend {
 public:
  // full_mesh = false: star (non-zero ranks connect only to rank 0), as the reference's TcpBackend.
  // full_mesh = true : every pair is connected (rank i listens on port+i, rank j>i connects to it), the gloo-native layout.
  TcpBackend(int rank, int world, const std::string& host, int port, bool full_mesh, int64_t connect_timeout_ms)
      : rank_(rank), world_(world), fds_(world, -1) {
    err_ = connect_all(host, port, full_mesh, connect_timeout_ms);
  }
  ~TcpBackend() override { close_all(); }
  int init_error() const { return err_; }
  int rank() const override { return rank_; }
  int world() const override { return world_; }

  int send(const void* data, size_t n, int dst) override {
    if (dst < 0 || dst >= world_) return E_INVALID_RANK;
    if (dst == rank_) return E_SELF_SEND;
    int f = fault.load();
    if (f == F_DROP_NEXT_SEND) { fault = F_NONE; return OK; }
    if (f == F_DELAY_SEND_MS) { fault = F_NONE; std::this_thread::sleep_for(std::chrono::milliseconds(fault_param.load())); }
    if (f == F_CLOSE) { fault = F_NONE; close_all(); return E_CHANNEL_CLOSED; }
    std::lock_guard<std::mutex> lk(send_mu_[dst % 8]);
    int fd = fds_[dst];
    if (fd < 0) return E_NO_CONNECTION;
    uint8_t hdr[8];
    put_u64le(hdr, f == F_CORRUPT_LENGTH ? (uint64_t)n + 1 : (uint64_t)n);
    if (f == F_CORRUPT_LENGTH) fault = F_NONE;
    // header and payload leave in one call: with TCP_NODELAY a separate 8-byte write would travel as a packet of its own
    iovec iov[2] = {{hdr, 8}, {const_cast<void*>(data), n}};
    msghdr msg{};
    msg.msg_iov = iov;
    msg.msg_iovlen = n ? 2 : 1;
    size_t left = 8 + n;
    while (left > 0) {
      ssize_t put = ::sendmsg(fd, &msg, MSG_NOSIGNAL);
      if (put < 0) { if (errno == EINTR) continue; return (errno == EPIPE || errno == ECONNRESET) ? E_CHANNEL_CLOSED : E_IO; }
      left -= (size_t)put;
      size_t adv = (size_t)put;
      while (adv > 0 && msg.msg_iovlen > 0) {
        if (adv >= msg.msg_iov[0].iov_len) { adv -= msg.msg_iov[0].iov_len; msg.msg_iov++; msg.msg_iovlen--; }
        else { msg.msg_iov[0].iov_base = (uint8_t*)msg.msg_iov[0].iov_base + adv; msg.msg_iov[0].iov_len -= adv; adv = 0; }
      }
    }
    return OK;
  }

  int recv(void* data, size_t n, int src, int64_t timeout_ms) override {
    if (src < 0 || src >= world_) return E_INVALID_RANK;
    if (src == rank_) return E_SELF_SEND;
    std::lock_guard<std::mutex> lk(recv_mu_[src % 8]);
    int fd = fds_[src];
    if (fd < 0) return E_NO_CONNECTION;
    uint8_t hdr[8];
    int e = read_full(fd, hdr, 8, timeout_ms);
    if (e) return e;
    uint64_t len = get_u64le(hdr);
    if (len != n) {
      // drain what the peer announced (bounded) so the stream stays framed, then report the mismatch
      std::vector<uint8_t> sink(std::min<uint64_t>(len, 1 << 20));
      uint64_t left = len;
      while (left > 0) { size_t c = (size_t)std::min<uint64_t>(left, sink.size()); if (read_full(fd, sink.data(), c, timeout_ms < 0 ? 1000 : timeout_ms)) break; left -= c; }
      return E_SIZE_MISMATCH;
    }
    return read_full(fd, data, n, timeout_ms);
  }

 private:
  // no Nagle delay; socket buffers large enough that a gradient bucket's send returns while the peer is still reducing the previous one
  static void tune_socket(int fd) {
    int one = 1, buf = 8 << 20;
    ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    ::setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
    ::setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
  }
  // The listener binds the rendezvous address itself (the one the peers connect to), not every interface: a rank announcement is all the
  // authentication the wire format has, so the port must not be reachable from networks the job does not use. FT_TCP_BIND_ANY=1 restores
  // the wildcard bind for hosts whose rendezvous address is a NAT or load-balancer address that no local interface carries.
  int listen_on(const std::string& host, int port, int* out_fd) {
    int fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) return E_IO;
    int one = 1;
    ::setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in a{};
    a.sin_family = AF_INET;
    const char* any = ::getenv("FT_TCP_BIND_ANY");
    if (any && any[0] == '1') a.sin_addr.s_addr = htonl(INADDR_ANY);
    else if (::inet_pton(AF_INET, host.c_str(), &a.sin_addr) != 1) { ::close(fd); return E_IO; }
    a.sin_port = htons((uint16_t)port);
    if (::bind(fd, (sockaddr*)&a, sizeof(a)) < 0 || ::listen(fd, 64) < 0) { ::close(fd); return E_IO; }
    *out_fd = fd;
    return OK;
  }
  int accept_peers(int lfd, int count, int64_t timeout_ms) {
    auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
    for (int i = 0; i < count; i++) {
      auto left = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - Clock::now()).count();
      if (left <= 0) return E_TIMEOUT;
      pollfd pfd{lfd, POLLIN, 0};
      int pr = ::poll(&pfd, 1, (int)left);
      if (pr <= 0) return pr == 0 ? E_TIMEOUT : E_IO;
      int fd = ::accept(lfd, nullptr, nullptr);
      if (fd < 0) return E_IO;
      tune_socket(fd);
      uint8_t hdr[8];
      int e = read_full(fd, hdr, 8, 5000);
      if (e) { ::close(fd); return e; }
      uint64_t peer = get_u64le(hdr);
      if (peer >= (uint64_t)world_ || fds_[peer] >= 0) { ::close(fd); return E_INVALID_RANK; }
      fds_[peer] = fd;
    }
    return OK;
  }
  int connect_to(const std::string& host, int port, int peer, int64_t timeout_ms) {
    auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_port = htons((uint16_t)port);
    if (::inet_pton(AF_INET, host.c_str(), &a.sin_addr) != 1) return E_IO;
    while (true) {
      int fd = ::socket(AF_INET, SOCK_STREAM, 0);
      if (fd < 0) return E_IO;
      if (::connect(fd, (sockaddr*)&a, sizeof(a)) == 0) {
        tune_socket(fd);
        uint8_t hdr[8];
        put_u64le(hdr, (uint64_t)rank_);
        int e = write_full(fd, hdr, 8);
        if (e) { ::close(fd); return e; }
        fds_[peer] = fd;
        return OK;
      }
      ::close(fd);
      if (Clock::now() >= deadline) return E_TIMEOUT;
      std::this_thread::sleep_for(std::chrono::milliseconds(50));   // rendezvous retry, 50 ms
    }
  }
  int connect_all(const std::string& host, int port, bool full_mesh, int64_t timeout_ms) {
    if (world_ < 1) return E_INVALID_WORLD;
    if (rank_ < 0 || rank_ >= world_) return E_INVALID_RANK;
    if (world_ == 1) return OK;
    if (!full_mesh) {
      if (rank_ == 0) {
        int lfd = -1, e = listen_on(host, port, &lfd);
        if (e) return e;
        e = accept_peers(lfd, world_ - 1, timeout_ms);
        ::close(lfd);
        return e;
      }
      return connect_to(host, port, 0, timeout_ms);
    }
    // full mesh: listen for higher ranks, connect to lower ranks
    int lfd = -1;
    if (rank_ < world_ - 1) { int e = listen_on(host, port + rank_, &lfd); if (e) return e; }
    for (int p = 0; p < rank_; p++) { int e = connect_to(host, port + p, p, timeout_ms); if (e) { if (lfd >= 0) ::close(lfd); return e; } }
    int e = OK;
    if (lfd >= 0) { e = accept_peers(lfd, world_ - 1 - rank_, timeout_ms); ::close(lfd); }
    return e;
  }
  void close_all() { for (int& fd : fds_) if (fd >= 0) { ::shutdown(fd, SHUT_RDWR); ::close(fd); fd = -1; } }

  int rank_, world_, err_ = OK;
  std::vector<int> fds_;
  std::mutex send_mu_[8], recv_mu_[8];
};

// ------------------------------------------------------------------------------------------------------------
// in-process fabric for thread ranks (the test fake; ferrotorch-distributed/src/backend.rs:395-569)
// ------------------------------------------------------------------------------------------------------------
struct SimFabric {
  explicit SimFabric(int n) : world(n), q(n * n) {}
  struct Chan { std::mutex mu; std::condition_variable cv; std::deque<std::vector<uint8_t>> msgs; bool closed = false; };
  int world;
  std::vector<Chan> q;   // q[src*world+dst]
};

class SimBackend : public Backend {
 public:
  SimBackend(std::shared_ptr<SimFabric> f, int rank) : f_(std::move(f)), rank_(rank) {}
  int rank() const override { return rank_; }
  int world() const override { return f_->world; }
  int send(const void* data, size_t n, int dst) override {
    if (dst < 0 || dst >= f_->world) return E_INVALID_RANK;
    if (dst == rank_) return E_SELF_SEND;
    int fl = fault.load();
    if (fl == F_DROP_NEXT_SEND) { fault = F_NONE; return OK; }
    if (fl == F_DELAY_SEND_MS) { fault = F_NONE; std::this_thread::sleep_for(std::chrono::milliseconds(fault_param.load())); }
    auto& c = f_->q[rank_ * f_->world + dst];
    if (fl == F_CLOSE) { fault = F_NONE; std::lock_guard<std::mutex> lk(c.mu); c.closed = true; c.cv.notify_all(); return E_CHANNEL_CLOSED; }
    std::vector<uint8_t> m(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + n);
    if (fl == F_CORRUPT_LENGTH) { fault = F_NONE; m.push_back(0); }
    { std::lock_guard<std::mutex> lk(c.mu); c.msgs.push_back(std::move(m)); }
    c.cv.notify_one();
    return OK;
  }
  int recv(void* data, size_t n, int src, int64_t timeout_ms) override {
    if (src < 0 || src >= f_->world) return E_INVALID_RANK;
    if (src == rank_) return E_SELF_SEND;
    auto& c = f_->q[src * f_->world + rank_];
    std::unique_lock<std::mutex> lk(c.mu);
    auto ready = [&] { return !c.msgs.empty() || c.closed; };
    if (timeout_ms < 0) c.cv.wait(lk, ready);
    else if (!c.cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), ready)) return E_TIMEOUT;
    if (c.msgs.empty()) return E_CHANNEL_CLOSED;
    std::vector<uint8_t> m = std::move(c.msgs.front());
    c.msgs.pop_front();
    if (m.size() != n) return E_SIZE_MISMATCH;
    if (n) std::memcpy(data, m.data(), n);
    return OK;
  }
 private:
  std::shared_ptr<SimFabric> f_;
  int rank_;
};

// sub-group view with a local<->global rank map (ferrotorch-distributed/src/backend.rs:595-753)
class SubBackend : public Backend {
 public:
  SubBackend(Backend* parent, std::vector<int> members) : parent_(parent), members_(std::move(members)) {
    local_ = -1;
    for (size_t i = 0; i < members_.size(); i++) if (members_[i] == parent_->rank()) local_ = (int)i;
  }
  bool valid() const { return local_ >= 0; }
  int rank() const override { return local_; }
  int world() const override { return (int)members_.size(); }
  int send(const void* d, size_t n, int dst) override {
    if (dst < 0 || dst >= world()) return E_INVALID_RANK;
    return parent_->send(d, n, members_[dst]);
  }
  int recv(void* d, size_t n, int src, int64_t t) override {
    if (src < 0 || src >= world()) return E_INVALID_RANK;
    return parent_->recv(d, n, members_[src], t);
  }
 private:
  Backend* parent_;
  std::vector<int> members_;
  int local_;
};

// ------------------------------------------------------------------------------------------------------------
// collectives over Backend
// ------------------------------------------------------------------------------------------------------------
enum DType : int { F32 = 0, F64 = 1 };
enum Op : int { SUM = 0, MEAN = 1, MAX = 2, MIN = 3, PROD = 4 };

template <typename T>
static void reduce_into(T* acc, const T* x, size_t n, int op) {
  switch (op) {
    case MAX: for (size_t i = 0; i < n; i++) acc[i] = std::max(acc[i], x[i]); break;
    case MIN: for (size_t i = 0; i < n; i++) acc[i] = std::min(acc[i], x[i]); break;
    case PROD: for (size_t i = 0; i < n; i++) acc[i] *= x[i]; break;
    default: for (size_t i = 0; i < n; i++) acc[i] += x[i];
  }
}

// Star all-reduce: rank 0 receives from ranks 1..N-1 in rank order, reduces in that order, applies the mean and sends the
// result back, so every rank ends up with bit-identical values.
template <typename T>
static int allreduce_star(Backend& b, T* data, size_t n, int op, int64_t timeout_ms) {
  const int r = b.rank(), w = b.world();
  if (w == 1) return OK;
  const size_t bytes = n * sizeof(T);
  // Large vectors go through in chunks so that the peers' uploads, the reduction on rank 0 and the downloads overlap: a peer sends its chunks
  // from a helper thread while its calling thread already receives reduced chunks. Element-wise the arithmetic (order of the ranks) is
  // that of the one-piece form, so the results stay bit-identical across ranks and across the two forms.
  constexpr size_t kChunkBytes = 256 << 10;
  if (bytes >= 8 * kChunkBytes) {   // from 2 MiB: below that the per-chunk frames cost more than the overlap saves
    const size_t ce = kChunkBytes / sizeof(T), nchunks = (n + ce - 1) / ce;
    if (r == 0) {
      std::vector<T> tmp(ce);
      for (size_t c = 0; c < nchunks; c++) {
        const size_t lo = c * ce, len = std::min(ce, n - lo);
        for (int p = 1; p < w; p++) {
          int e = b.recv(tmp.data(), len * sizeof(T), p, timeout_ms);
          if (e) return e;
          reduce_into(data + lo, tmp.data(), len, op);
        }
        if (op == MEAN) { const T inv = (T)w; for (size_t i = 0; i < len; i++) data[lo + i] /= inv; }
        for (int p = 1; p < w; p++) { int e = b.send(data + lo, len * sizeof(T), p); if (e) return e; }
      }
      return OK;
    }
    std::atomic<size_t> sent{0};
    std::atomic<int> send_err{OK};
    std::thread sender([&] {
      for (size_t c = 0; c < nchunks; c++) {
        const size_t lo = c * ce, len = std::min(ce, n - lo);
        int e = b.send(data + lo, len * sizeof(T), 0);
        if (e) { send_err.store(e, std::memory_order_release); return; }
        sent.store(c + 1, std::memory_order_release);
      }
    });
    int err = OK;
    for (size_t c = 0; c < nchunks && !err; c++) {
      const size_t lo = c * ce, len = std::min(ce, n - lo);
      // chunk c comes back only after it went out; the wait makes that order visible to this thread before it overwrites the chunk
      while (sent.load(std::memory_order_acquire) <= c && !(err = send_err.load(std::memory_order_acquire))) std::this_thread::yield();
      if (!err) err = b.recv(data + lo, len * sizeof(T), 0, timeout_ms);
    }
    sender.join();
    return err ? err : send_err.load();
  }
  if (r == 0) {
    std::vector<T> tmp(n);
    for (int p = 1; p < w; p++) {
      int e = b.recv(tmp.data(), bytes, p, timeout_ms);
      if (e) return e;
      reduce_into(data, tmp.data(), n, op);
    }
    if (op == MEAN) { const T inv = (T)w; for (size_t i = 0; i < n; i++) data[i] /= inv; }
    for (int p = 1; p < w; p++) { int e = b.send(data, bytes, p); if (e) return e; }
    return OK;
  }
  int e = b.send(data, bytes, 0);
  if (e) return e;
  return b.recv(data, bytes, 0, timeout_ms);
}

// Ring all-reduce (every reduce op): chunk i = [i*n/N, (i+1)*n/N); N-1 reduce-scatter steps then N-1 all-gather steps;
// needs a backend where neighbours are connected (full mesh TCP or the simulated fabric).
template <typename T>
static int allreduce_ring(Backend& b, T* data, size_t n, int op, int64_t timeout_ms) {
  const int r = b.rank(), w = b.world();
  if (w == 1) return OK;
  if (op < SUM || op > PROD) return E_UNSUPPORTED;
  auto lo = [&](int i) { return (size_t)((uint64_t)n * (uint64_t)i / (uint64_t)w); };
  const int next = (r + 1) % w, prev = (r + w - 1) % w;
  std::vector<T> tmp(n / w + 2);
  auto exchange = [&](const T* sbuf, size_t sn, T* rbuf, size_t rn) -> int {
    // even ranks send first, odd ranks receive first: no deadlock on rendezvous-less transports
    int e;
    if (r % 2 == 0) { e = b.send(sbuf, sn * sizeof(T), next); if (e) return e; e = b.recv(rbuf, rn * sizeof(T), prev, timeout_ms); }
    else { e = b.recv(rbuf, rn * sizeof(T), prev, timeout_ms); if (e) return e; e = b.send(sbuf, sn * sizeof(T), next); }
    return e;
  };
  for (int s = 0; s < w - 1; s++) {
    const int sc = (r - s + w) % w, rc = (r - s - 1 + w) % w;
    int e = exchange(data + lo(sc), lo(sc + 1) - lo(sc), tmp.data(), lo(rc + 1) - lo(rc));
    if (e) return e;
    reduce_into(data + lo(rc), tmp.data(), lo(rc + 1) - lo(rc), op);
  }
  for (int s = 0; s < w - 1; s++) {
    const int sc = (r + 1 - s + w) % w, rc = (r - s + w) % w;
    int e = exchange(data + lo(sc), lo(sc + 1) - lo(sc), data + lo(rc), lo(rc + 1) - lo(rc));
    if (e) return e;
  }
  if (op == MEAN) { const T inv = (T)w; for (size_t i = 0; i < n; i++) data[i] /= inv; }
  return OK;
}

static int broadcast_star(Backend& b, void* data, size_t bytes, int root, int64_t timeout_ms) {
  const int r = b.rank(), w = b.world();
  if (root < 0 || root >= w) return E_INVALID_RANK;
  if (w == 1) return OK;
  if (r == root) { for (int p = 0; p < w; p++) if (p != root) { int e = b.send(data, bytes, p); if (e) return e; } return OK; }
  return b.recv(data, bytes, root, timeout_ms);
}

// binomial tree broadcast (gloo-native style); requires full connectivity
static int broadcast_tree(Backend& b, void* data, size_t bytes, int root, int64_t timeout_ms) {
  const int w = b.world(), vr = (b.rank() - root + w) % w;
  int mask = 1;
  while (mask < w) {
    if (vr & mask) { int src = (vr - mask + root) % w; int e = b.recv(data, bytes, src, timeout_ms); if (e) return e; break; }
    mask <<= 1;
  }
  mask >>= 1;
  while (mask > 0) {
    if (vr + mask < w) { int dst = (vr + mask + root) % w; int e = b.send(data, bytes, dst); if (e) return e; }
    mask >>= 1;
  }
  return OK;
}

// all-gather of equal-size byte blocks through rank 0 (gather, then re-broadcast of the concatenation)
static int all_gather_star(Backend& b, const void* mine, size_t bytes, void* out, int64_t timeout_ms) {
  const int r = b.rank(), w = b.world();
  uint8_t* o = static_cast<uint8_t*>(out);
  if (w == 1) { std::memcpy(o, mine, bytes); return OK; }
  if (r == 0) {
    std::memcpy(o, mine, bytes);
    for (int p = 1; p < w; p++) { int e = b.recv(o + (size_t)p * bytes, bytes, p, timeout_ms); if (e) return e; }
    for (int p = 1; p < w; p++) { int e = b.send(o, bytes * w, p); if (e) return e; }
    return OK;
  }
  int e = b.send(mine, bytes, 0);
  if (e) return e;
  return b.recv(o, bytes * w, 0, timeout_ms);
}

// reduce-scatter through rank 0: full[n*w] -> out[n] = reduce over ranks of full[rank*n : (rank+1)*n]
template <typename T>
static int reduce_scatter_star(Backend& b, const T* full, size_t chunk, T* out, int op, int64_t timeout_ms) {
  const int r = b.rank(), w = b.world();
  if (w == 1) { std::memcpy(out, full, chunk * sizeof(T)); return OK; }
  const size_t n = chunk * w;
  if (r == 0) {
    std::vector<T> acc(full, full + n), tmp(n);
    for (int p = 1; p < w; p++) { int e = b.recv(tmp.data(), n * sizeof(T), p, timeout_ms); if (e) return e; reduce_into(acc.data(), tmp.data(), n, op); }
    if (op == MEAN) { const T inv = (T)w; for (auto& v : acc) v /= inv; }
    std::memcpy(out, acc.data(), chunk * sizeof(T));
    for (int p = 1; p < w; p++) { int e = b.send(acc.data() + (size_t)p * chunk, chunk * sizeof(T), p); if (e) return e; }
    return OK;
  }
  int e = b.send(full, n * sizeof(T), 0);
  if (e) return e;
  return b.recv(out, chunk * sizeof(T), 0, timeout_ms);
}

// pairwise all-to-all with per-peer byte counts; the lower rank of each pair sends first (collective.rs:457-651).
// On a star transport non-zero ranks cannot reach each other: E_NO_CONNECTION is returned for those pairs.
static int all_to_all(Backend& b, const uint8_t* send, const int64_t* send_counts, uint8_t* recv, const int64_t* recv_counts,
                      int64_t timeout_ms) {
  const int r = b.rank(), w = b.world();
  std::vector<size_t> soff(w + 1, 0), roff(w + 1, 0);
  for (int p = 0; p < w; p++) { soff[p + 1] = soff[p] + (size_t)send_counts[p]; roff[p + 1] = roff[p] + (size_t)recv_counts[p]; }
  std::memcpy(recv + roff[r], send + soff[r], (size_t)send_counts[r]);
  for (int p = 0; p < w; p++) {
    if (p == r) continue;
    int e;
    if (r < p) {
      e = b.send(send + soff[p], (size_t)send_counts[p], p); if (e) return e;
      e = b.recv(recv + roff[p], (size_t)recv_counts[p], p, timeout_ms); if (e) return e;
    } else {
      e = b.recv(recv + roff[p], (size_t)recv_counts[p], p, timeout_ms); if (e) return e;
      e = b.send(send + soff[p], (size_t)send_counts[p], p); if (e) return e;
    }
  }
  return OK;
}

// ------------------------------------------------------------------------------------------------------------
// handle registry
// ------------------------------------------------------------------------------------------------------------
static std::mutex g_mu;
static std::map<int64_t, std::shared_ptr<Backend>> g_backends;
static std::map<int64_t, std::shared_ptr<SimFabric>> g_fabrics;
static int64_t g_next = 1;

static std::shared_ptr<Backend> get(int64_t h) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_backends.find(h);
  return it == g_backends.end() ? nullptr : it->second;
}

}  // namespace ft

using namespace ft;

FT_API int64_t ft_tcp_backend_create(int rank, int world, const char* host, int port, int full_mesh, int64_t connect_timeout_ms, int* err) {
  auto b = std::make_shared<TcpBackend>(rank, world, host ? host : "127.0.0.1", port, full_mesh != 0, connect_timeout_ms);
  if (b->init_error()) { if (err) *err = b->init_error(); return 0; }
  if (err) *err = OK;
  std::lock_guard<std::mutex> lk(g_mu);
  g_backends[g_next] = b;
  return g_next++;
}

FT_API int64_t ft_sim_fabric_create(int world) {
  if (world < 1) return 0;
  std::lock_guard<std::mutex> lk(g_mu);
  g_fabrics[g_next] = std::make_shared<SimFabric>(world);
  return g_next++;
}

FT_API int64_t ft_sim_backend_create(int64_t fabric, int rank) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_fabrics.find(fabric);
  if (it == g_fabrics.end() || rank < 0 || rank >= it->second->world) return 0;
  g_backends[g_next] = std::make_shared<SimBackend>(it->second, rank);
  return g_next++;
}

FT_API int64_t ft_sub_backend_create(int64_t parent, const int* members, int n) {
  auto p = get(parent);
  if (!p || n < 1) return 0;
  for (int i = 0; i < n; i++) if (members[i] < 0 || members[i] >= p->world()) return 0;
  auto sb = std::make_shared<SubBackend>(p.get(), std::vector<int>(members, members + n));
  if (!sb->valid()) return 0;
  std::lock_guard<std::mutex> lk(g_mu);
  g_backends[g_next] = sb;
  g_backends[-g_next] = p;   // keep the parent alive as long as the view exists
  return g_next++;
}

FT_API void ft_backend_destroy(int64_t h) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_backends.erase(h);
  g_backends.erase(-h);
  g_fabrics.erase(h);
}

FT_API int ft_backend_rank(int64_t h) { auto b = get(h); return b ? b->rank() : -1; }
FT_API int ft_backend_world(int64_t h) { auto b = get(h); return b ? b->world() : -1; }
FT_API int ft_backend_send(int64_t h, const void* d, int64_t n, int dst) { auto b = get(h); return b ? b->send(d, (size_t)n, dst) : E_ARG; }
FT_API int ft_backend_recv(int64_t h, void* d, int64_t n, int src, int64_t timeout_ms) { auto b = get(h); return b ? b->recv(d, (size_t)n, src, timeout_ms) : E_ARG; }
FT_API int ft_backend_barrier(int64_t h, int64_t timeout_ms) { auto b = get(h); return b ? b->barrier(timeout_ms) : E_ARG; }
FT_API int ft_backend_set_fault(int64_t h, int kind, int64_t param) {
  auto b = get(h);
  if (!b) return E_ARG;
  b->fault_param = param;
  b->fault = kind;
  return OK;
}

// algo: 0 star, 1 ring. dtype: 0 f32, 1 f64. op: 0 sum, 1 mean, 2 max, 3 min, 4 prod.
FT_API int ft_allreduce(int64_t h, void* data, int64_t n, int dtype, int op, int algo, int64_t timeout_ms) {
  auto b = get(h);
  if (!b || n < 0) return E_ARG;
  if (n == 0) return OK;
  if (dtype == F32) return algo == 1 ? allreduce_ring(*b, (float*)data, (size_t)n, op, timeout_ms) : allreduce_star(*b, (float*)data, (size_t)n, op, timeout_ms);
  if (dtype == F64) return algo == 1 ? allreduce_ring(*b, (double*)data, (size_t)n, op, timeout_ms) : allreduce_star(*b, (double*)data, (size_t)n, op, timeout_ms);
  return E_UNSUPPORTED;
}
FT_API int ft_broadcast(int64_t h, void* data, int64_t bytes, int root, int algo, int64_t timeout_ms) {
  auto b = get(h);
  if (!b || bytes < 0) return E_ARG;
  if (bytes == 0) return OK;
  return algo == 1 ? broadcast_tree(*b, data, (size_t)bytes, root, timeout_ms) : broadcast_star(*b, data, (size_t)bytes, root, timeout_ms);
}
FT_API int ft_all_gather(int64_t h, const void* mine, int64_t bytes, void* out, int64_t timeout_ms) {
  auto b = get(h);
  if (!b || bytes < 0) return E_ARG;
  if (bytes == 0) return OK;
  return all_gather_star(*b, mine, (size_t)bytes, out, timeout_ms);
}
FT_API int ft_reduce_scatter(int64_t h, const void* full, int64_t chunk, void* out, int dtype, int op, int64_t timeout_ms) {
  auto b = get(h);
  if (!b || chunk < 0) return E_ARG;
  if (chunk == 0) return OK;
  if (dtype == F32) return reduce_scatter_star(*b, (const float*)full, (size_t)chunk, (float*)out, op, timeout_ms);
  if (dtype == F64) return reduce_scatter_star(*b, (const double*)full, (size_t)chunk, (double*)out, op, timeout_ms);
  return E_UNSUPPORTED;
}
FT_API int ft_all_to_all(int64_t h, const void* send, const int64_t* send_counts, void* recv, const int64_t* recv_counts, int64_t timeout_ms) {
  auto b = get(h);
  if (!b) return E_ARG;
  return all_to_all(*b, (const uint8_t*)send, send_counts, (uint8_t*)recv, recv_counts, timeout_ms);
}

// DDP bucket plan: parameters are walked in reverse order and packed greedily into buckets of at most cap_bytes
// (a parameter larger than the cap gets a bucket of its own). bucket_of[i] receives the bucket index of parameter i.
// Returns the number of buckets. (ferrotorch-distributed/src/ddp.rs:213-241)
FT_API int ft_ddp_plan_buckets(const int64_t* numels, int n_params, int elem_bytes, int64_t cap_bytes, int* bucket_of) {
  int bucket = 0;
  int64_t cur = 0;
  bool any = false;
  for (int i = n_params - 1; i >= 0; i--) {
    const int64_t bytes = numels[i] * elem_bytes;
    if (any && cur + bytes > cap_bytes) { bucket++; cur = 0; any = false; }
    bucket_of[i] = bucket;
    cur += bytes;
    any = true;
  }
  return n_params > 0 ? bucket + 1 : 0;
}

FT_API int ft_runtime_abi_version() { return 1; }
