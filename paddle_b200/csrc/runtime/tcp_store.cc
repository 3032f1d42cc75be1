// TCP key-value store for rendezvous (reference: paddle/phi/core/distributed/store/tcp_store.h:40-139,
// tcp_store.cc).  Rank 0 runs a master daemon thread with a poll() loop; clients send framed commands
// SET / GET / ADD / CHECK / WAIT / DELETE / STOP over one persistent connection each.  GET and WAIT block
// on the server side until the key exists (or the client-side timeout closes the socket).
// Exposed through a C ABI (pd_store_*) and used by paddle_b200.distributed.store.TCPStore.
#include <arpa/inet.h>
#include <errno.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#define PD_EXPORT extern "C" __attribute__((visibility("default")))

namespace pdrt {

enum Cmd : uint8_t { kSet = 1, kGet = 2, kAdd = 3, kCheck = 4, kWait = 5, kDelete = 6, kStop = 7 };

static bool send_all(int fd, const void* buf, size_t n) {
  const char* p = static_cast<const char*>(buf);
  while (n > 0) {
    ssize_t k = ::send(fd, p, n, MSG_NOSIGNAL);
    if (k <= 0) {
      if (k < 0 && (errno == EINTR)) continue;
      return false;
    }
    p += k;
    n -= static_cast<size_t>(k);
  }
  return true;
}
static bool recv_all(int fd, void* buf, size_t n) {
  char* p = static_cast<char*>(buf);
  while (n > 0) {
    ssize_t k = ::recv(fd, p, n, 0);
    if (k <= 0) {
      if (k < 0 && (errno == EINTR)) continue;
      return false;
    }
    p += k;
    n -= static_cast<size_t>(k);
  }
  return true;
}
static bool send_blob(int fd, const std::string& s) {
  uint64_t n = s.size();
  return send_all(fd, &n, 8) && (n == 0 || send_all(fd, s.data(), n));
}
static bool recv_blob(int fd, std::string* s) {
  uint64_t n = 0;
  if (!recv_all(fd, &n, 8)) return false;
  if (n > (1ull << 31)) return false;
  s->resize(n);
  return n == 0 || recv_all(fd, &(*s)[0], n);
}

class MasterDaemon {
 public:
  explicit MasterDaemon(int listen_fd) : listen_fd_(listen_fd), stop_(false) {
    thread_ = std::thread([this] { Run(); });
  }
  ~MasterDaemon() {
    stop_ = true;
    if (thread_.joinable()) thread_.join();
    for (int fd : clients_) ::close(fd);
    ::close(listen_fd_);
  }

 private:
  struct Waiter {
    int fd;
    std::string key;
    bool want_value;
  };
  void Reply(const Waiter& w) {
    if (w.want_value) {
      send_blob(w.fd, kv_[w.key]);
    } else {
      uint8_t ok = 1;
      send_all(w.fd, &ok, 1);
    }
  }
  void WakeWaiters(const std::string& key) {
    std::vector<Waiter> rest;
    for (auto& w : waiters_) {
      if (w.key == key) Reply(w); else rest.push_back(w);
    }
    waiters_.swap(rest);
  }
  bool Handle(int fd) {
    uint8_t cmd;
    if (!recv_all(fd, &cmd, 1)) return false;
    std::string key;
    if (cmd != kStop && !recv_blob(fd, &key)) return false;
    switch (cmd) {
      case kSet: {
        std::string val;
        if (!recv_blob(fd, &val)) return false;
        kv_[key] = val;
        WakeWaiters(key);
        return true;
      }
      case kGet:
      case kWait: {
        Waiter w{fd, key, cmd == kGet};
        if (kv_.count(key)) Reply(w); else waiters_.push_back(w);
        return true;
      }
      case kAdd: {
        int64_t delta;
        if (!recv_all(fd, &delta, 8)) return false;
        int64_t cur = 0;
        auto it = kv_.find(key);
        if (it != kv_.end() && it->second.size() == 8) memcpy(&cur, it->second.data(), 8);
        cur += delta;
        kv_[key] = std::string(reinterpret_cast<char*>(&cur), 8);
        send_all(fd, &cur, 8);
        WakeWaiters(key);
        return true;
      }
      case kCheck: {
        uint8_t has = kv_.count(key) ? 1 : 0;
        return send_all(fd, &has, 1);
      }
      case kDelete: {
        uint8_t had = kv_.erase(key) ? 1 : 0;
        return send_all(fd, &had, 1);
      }
      case kStop:
        stop_ = true;
        return true;
      default:
        return false;
    }
  }
  void Run() {
    while (!stop_) {
      std::vector<pollfd> fds;
      fds.push_back({listen_fd_, POLLIN, 0});
      for (int fd : clients_) fds.push_back({fd, POLLIN, 0});
      int n = ::poll(fds.data(), fds.size(), 100);
      if (n <= 0) continue;
      if (fds[0].revents & POLLIN) {
        int c = ::accept(listen_fd_, nullptr, nullptr);
        if (c >= 0) {
          int one = 1;
          setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
          clients_.push_back(c);
        }
      }
      std::vector<int> dead;
      for (size_t i = 1; i < fds.size(); ++i) {
        if (fds[i].revents & (POLLIN | POLLHUP | POLLERR)) {
          if (!Handle(fds[i].fd)) dead.push_back(fds[i].fd);
        }
      }
      for (int fd : dead) {
        ::close(fd);
        for (size_t i = 0; i < clients_.size(); ++i)
          if (clients_[i] == fd) { clients_.erase(clients_.begin() + i); break; }
        std::vector<Waiter> rest;
        for (auto& w : waiters_) if (w.fd != fd) rest.push_back(w);
        waiters_.swap(rest);
      }
    }
  }
  int listen_fd_;
  std::atomic<bool> stop_;
  std::thread thread_;
  std::vector<int> clients_;
  std::unordered_map<std::string, std::string> kv_;
  std::vector<Waiter> waiters_;
};

struct Store {
  int fd = -1;
  MasterDaemon* daemon = nullptr;
  int timeout_ms = 900000;
  std::mutex mu;
};

static int connect_with_retry(const char* host, int port, int timeout_ms) {
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  char portstr[16];
  snprintf(portstr, sizeof(portstr), "%d", port);
  while (std::chrono::steady_clock::now() < deadline) {
    addrinfo hints{}, *res = nullptr;
    hints.ai_family = AF_INET;
    hints.ai_socktype = SOCK_STREAM;
    if (getaddrinfo(host, portstr, &hints, &res) == 0 && res) {
      int fd = ::socket(res->ai_family, res->ai_socktype, res->ai_protocol);
      if (fd >= 0) {
        if (::connect(fd, res->ai_addr, res->ai_addrlen) == 0) {
          int one = 1;
          setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
          freeaddrinfo(res);
          return fd;
        }
        ::close(fd);
      }
      freeaddrinfo(res);
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(50));
  }
  return -1;
}

static bool wait_readable(int fd, int timeout_ms) {
  pollfd p{fd, POLLIN, 0};
  return ::poll(&p, 1, timeout_ms) > 0;
}

}  // namespace pdrt

using namespace pdrt;

// Returns an opaque handle or null.  is_master: bind + serve on `port` (0 = pick a free one, see pd_store_port).
PD_EXPORT void* pd_store_create(const char* host, int port, int is_master, int timeout_ms) {
  Store* s = new Store();
  s->timeout_ms = timeout_ms;
  if (is_master) {
    int lfd = ::socket(AF_INET, SOCK_STREAM, 0);
    int one = 1;
    setsockopt(lfd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_addr.s_addr = htonl(INADDR_ANY);
    addr.sin_port = htons(static_cast<uint16_t>(port));
    if (::bind(lfd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(lfd, 512) != 0) {
      ::close(lfd);
      delete s;
      return nullptr;
    }
    socklen_t len = sizeof(addr);
    getsockname(lfd, reinterpret_cast<sockaddr*>(&addr), &len);
    port = ntohs(addr.sin_port);
    s->daemon = new MasterDaemon(lfd);
  }
  s->fd = connect_with_retry(is_master ? "127.0.0.1" : host, port, timeout_ms);
  if (s->fd < 0) {
    delete s->daemon;
    delete s;
    return nullptr;
  }
  // remember the port for pd_store_port
  sockaddr_in peer{};
  socklen_t len = sizeof(peer);
  getpeername(s->fd, reinterpret_cast<sockaddr*>(&peer), &len);
  return s;
}
PD_EXPORT int pd_store_port(void* h) {
  Store* s = static_cast<Store*>(h);
  sockaddr_in peer{};
  socklen_t len = sizeof(peer);
  getpeername(s->fd, reinterpret_cast<sockaddr*>(&peer), &len);
  return ntohs(peer.sin_port);
}
PD_EXPORT void pd_store_destroy(void* h) {
  Store* s = static_cast<Store*>(h);
  if (!s) return;
  if (s->fd >= 0) ::close(s->fd);
  delete s->daemon;
  delete s;
}
PD_EXPORT int pd_store_set(void* h, const char* key, const void* val, int64_t n) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  uint8_t cmd = kSet;
  return send_all(s->fd, &cmd, 1) && send_blob(s->fd, key) &&
                 send_blob(s->fd, std::string(static_cast<const char*>(val), static_cast<size_t>(n))) ? 0 : -1;
}
// Blocks until the key exists or timeout.  Returns the value length (copied into buf up to cap), -1 on
// error, -2 on timeout (the connection is then unusable and is closed).
PD_EXPORT int64_t pd_store_get(void* h, const char* key, void* buf, int64_t cap) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  uint8_t cmd = kGet;
  if (!send_all(s->fd, &cmd, 1) || !send_blob(s->fd, key)) return -1;
  if (!wait_readable(s->fd, s->timeout_ms)) {
    ::close(s->fd);
    s->fd = -1;
    return -2;
  }
  std::string val;
  if (!recv_blob(s->fd, &val)) return -1;
  memcpy(buf, val.data(), static_cast<size_t>(std::min<int64_t>(cap, static_cast<int64_t>(val.size()))));
  return static_cast<int64_t>(val.size());
}
PD_EXPORT int64_t pd_store_add(void* h, const char* key, int64_t delta) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  uint8_t cmd = kAdd;
  int64_t out = 0;
  if (!send_all(s->fd, &cmd, 1) || !send_blob(s->fd, key) || !send_all(s->fd, &delta, 8) || !recv_all(s->fd, &out, 8))
    return INT64_MIN;
  return out;
}
PD_EXPORT int pd_store_check(void* h, const char* key) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  uint8_t cmd = kCheck, has = 0;
  if (!send_all(s->fd, &cmd, 1) || !send_blob(s->fd, key) || !recv_all(s->fd, &has, 1)) return -1;
  return has;
}
PD_EXPORT int pd_store_delete(void* h, const char* key) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  uint8_t cmd = kDelete, had = 0;
  if (!send_all(s->fd, &cmd, 1) || !send_blob(s->fd, key) || !recv_all(s->fd, &had, 1)) return -1;
  return had;
}
// 0 = key present, -2 = timeout (connection closed), -1 = error
PD_EXPORT int pd_store_wait(void* h, const char* key, int timeout_ms) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  uint8_t cmd = kWait, ok = 0;
  if (!send_all(s->fd, &cmd, 1) || !send_blob(s->fd, key)) return -1;
  if (!wait_readable(s->fd, timeout_ms > 0 ? timeout_ms : s->timeout_ms)) {
    ::close(s->fd);
    s->fd = -1;
    return -2;
  }
  return recv_all(s->fd, &ok, 1) ? 0 : -1;
}
