#include "core/util.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <pthread.h>
#include <sys/socket.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>

#include "core/log.h"

namespace kvx {

void SyncSemaphore::wait(uint32_t cond) {
  // Layers of a step are usually signalled a few microseconds apart: spin briefly (a sleeping
  // waiter costs a futex wake-up per layer), then block.
  for (int i = 0; i < 1000; ++i) {
    if (fast_.load(std::memory_order_acquire) > cond) return;
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
  }
  std::unique_lock<std::mutex> lk(mu_);
  cv_.wait(lk, [&] { return ready_ > cond; });
}

bool SyncSemaphore::wait_for(uint32_t cond, std::chrono::milliseconds timeout) {
  std::unique_lock<std::mutex> lk(mu_);
  return cv_.wait_for(lk, timeout, [&] { return ready_ > cond; });
}

void SyncSemaphore::release() {
  {
    std::lock_guard<std::mutex> g(mu_);
    ++ready_;
    fast_.store(ready_, std::memory_order_release);
  }
  cv_.notify_all();
}

uint32_t SyncSemaphore::release(uint32_t cond) {
  uint32_t v;
  {
    std::lock_guard<std::mutex> g(mu_);
    if (ready_ < cond) ready_ = cond;
    v = ready_;
    fast_.store(ready_, std::memory_order_release);
  }
  cv_.notify_all();
  return v;
}

uint32_t SyncSemaphore::value() {
  std::lock_guard<std::mutex> g(mu_);
  return ready_;
}

ThreadPool::ThreadPool(size_t n, std::string name) : name_(std::move(name)) {
  if (n == 0) n = 1;
  for (size_t i = 0; i < n; ++i) {
    workers_.emplace_back(std::make_unique<Worker>());
    Worker* w = workers_.back().get();
    w->thd = std::thread([this, w, i] { run(w, i); });
  }
}

ThreadPool::~ThreadPool() {
  stop_.store(true);
  for (auto& w : workers_) {
    {
      std::lock_guard<std::mutex> g(w->mu);
    }
    w->cv.notify_all();
  }
  for (auto& w : workers_)
    if (w->thd.joinable()) w->thd.join();
}

void ThreadPool::run(Worker* w, size_t idx) {
  std::string nm = name_ + std::to_string(idx);
  pthread_setname_np(pthread_self(), nm.substr(0, 15).c_str());
  for (;;) {
    std::function<void()> fn;
    {
      std::unique_lock<std::mutex> lk(w->mu);
      w->busy = false;
      w->cv.notify_all();
      w->cv.wait(lk, [&] { return stop_.load() || !w->q.empty(); });
      if (w->q.empty()) return;  // stopping and drained
      fn = std::move(w->q.front());
      w->q.pop_front();
      w->busy = true;
    }
    try {
      fn();
    } catch (const std::exception& ex) {
      LOG(ERROR) << "thread pool task threw: " << ex.what();
    } catch (...) {
      LOG(ERROR) << "thread pool task threw a non-std exception";
    }
    w->pending.fetch_sub(1, std::memory_order_release);
  }
}

void ThreadPool::spawn(std::function<void()> fn) {
  // least-loaded of two round-robin candidates keeps unrelated tasks from queueing behind a long one
  size_t a = rr_.fetch_add(1) % workers_.size();
  spawn(std::move(fn), static_cast<int>(a));
}

void ThreadPool::spawn(std::function<void()> fn, int hint) {
  Worker* w = workers_[static_cast<size_t>(hint < 0 ? -hint : hint) % workers_.size()].get();
  {
    std::lock_guard<std::mutex> g(w->mu);
    w->pending.fetch_add(1, std::memory_order_relaxed);
    w->q.emplace_back(std::move(fn));
  }
  w->cv.notify_all();
}

void ThreadPool::drain() {
  // A caller that drains is about to use the result: poll for a short while (a sleeping thread is
  // woken some tens of microseconds after the notify), then block.
  const auto t0 = std::chrono::steady_clock::now();
  for (auto& w : workers_) {
    while (w->pending.load(std::memory_order_acquire) != 0) {
      if (std::chrono::steady_clock::now() - t0 > std::chrono::microseconds(500)) break;
      __builtin_ia32_pause();
    }
    if (w->pending.load(std::memory_order_acquire) == 0) continue;
    std::unique_lock<std::mutex> lk(w->mu);
    w->cv.wait(lk, [&] { return w->pending.load(std::memory_order_acquire) == 0; });
  }
}

FdGuard& FdGuard::operator=(FdGuard&& o) noexcept {
  if (this != &o) {
    reset();
    fd_ = o.fd_;
    o.fd_ = -1;
  }
  return *this;
}
FdGuard::~FdGuard() { reset(); }
void FdGuard::reset() {
  if (fd_ >= 0) ::close(fd_);
  fd_ = -1;
}

static int wait_fd(int fd, short events, int timeout_ms) {
  struct pollfd p;
  p.fd = fd;
  p.events = events;
  p.revents = 0;
  for (;;) {
    int r = ::poll(&p, 1, timeout_ms > 0 ? timeout_ms : -1);
    if (r < 0 && errno == EINTR) continue;
    if (r == 0) {
      errno = ETIMEDOUT;
      return -1;
    }
    return r;
  }
}

int tcp_connect(const std::string& ip, int port, int timeout_ms) {
  int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return -1;
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (inet_pton(AF_INET, ip.c_str(), &addr.sin_addr) != 1) {
    ::close(fd);
    errno = EINVAL;
    return -1;
  }
  int flags = fcntl(fd, F_GETFL, 0);
  fcntl(fd, F_SETFL, flags | O_NONBLOCK);
  int r = ::connect(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr));
  if (r < 0 && errno != EINPROGRESS) {
    int e = errno;
    ::close(fd);
    errno = e;
    return -1;
  }
  if (r < 0) {
    if (wait_fd(fd, POLLOUT, timeout_ms) < 0) {
      int e = errno;
      ::close(fd);
      errno = e;
      return -1;
    }
    int err = 0;
    socklen_t len = sizeof(err);
    getsockopt(fd, SOL_SOCKET, SO_ERROR, &err, &len);
    if (err != 0) {
      ::close(fd);
      errno = err;
      return -1;
    }
  }
  fcntl(fd, F_SETFL, flags);
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  return fd;
}

int tcp_listen(const std::string& ip, int port, int backlog, int* bound_port) {
  int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return -1;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (ip.empty() || ip == "0.0.0.0") addr.sin_addr.s_addr = htonl(INADDR_ANY);
  else if (inet_pton(AF_INET, ip.c_str(), &addr.sin_addr) != 1) {
    ::close(fd);
    errno = EINVAL;
    return -1;
  }
  if (::bind(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) < 0 || ::listen(fd, backlog) < 0) {
    int e = errno;
    ::close(fd);
    errno = e;
    return -1;
  }
  if (bound_port != nullptr) {
    socklen_t len = sizeof(addr);
    getsockname(fd, reinterpret_cast<sockaddr*>(&addr), &len);
    *bound_port = ntohs(addr.sin_port);
  }
  return fd;
}

ssize_t write_full(int fd, const void* buf, size_t len, int timeout_ms) {
  const char* p = static_cast<const char*>(buf);
  size_t done = 0;
  while (done < len) {
    ssize_t r = ::send(fd, p + done, len - done, MSG_NOSIGNAL);
    if (r < 0) {
      if (errno == EINTR) continue;
      if (errno == EAGAIN || errno == EWOULDBLOCK) {
        if (wait_fd(fd, POLLOUT, timeout_ms) < 0) return -1;
        continue;
      }
      return -1;
    }
    done += static_cast<size_t>(r);
  }
  return static_cast<ssize_t>(done);
}

ssize_t read_full(int fd, void* buf, size_t len, int timeout_ms) {
  char* p = static_cast<char*>(buf);
  size_t done = 0;
  while (done < len) {
    if (timeout_ms > 0 && wait_fd(fd, POLLIN, timeout_ms) < 0) return -1;
    ssize_t r = ::recv(fd, p + done, len - done, 0);
    if (r == 0) return static_cast<ssize_t>(done);  // peer closed
    if (r < 0) {
      if (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK) continue;
      return -1;
    }
    done += static_cast<size_t>(r);
  }
  return static_cast<ssize_t>(done);
}

std::string local_ip() {
  const char* env = getenv("VLLM_HOST_IP");
  if (env != nullptr && *env != '\0') return env;
  int fd = ::socket(AF_INET, SOCK_DGRAM, 0);
  if (fd < 0) return "127.0.0.1";
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = htons(80);
  inet_pton(AF_INET, "8.8.8.8", &addr.sin_addr);
  std::string out = "127.0.0.1";
  if (::connect(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) == 0) {
    sockaddr_in me{};
    socklen_t len = sizeof(me);
    if (getsockname(fd, reinterpret_cast<sockaddr*>(&me), &len) == 0) {
      char buf[64];
      if (inet_ntop(AF_INET, &me.sin_addr, buf, sizeof(buf)) != nullptr) out = buf;
    }
  }
  ::close(fd);
  return out;
}

}  // namespace kvx
