// Small building blocks: monotone semaphore, thread pools, blocking queue, timers, sockets.
#pragma once
#include <sys/types.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <thread>
#include <vector>

namespace kvx {

using SteadyClock = std::chrono::steady_clock;
using Timepoint = SteadyClock::time_point;

inline int64_t elapse_us(Timepoint a, Timepoint b) {
  return std::chrono::duration_cast<std::chrono::microseconds>(b - a).count();
}

class TimeWatch {
 public:
  TimeWatch() : start_(SteadyClock::now()) {}
  int64_t get_elapse_us() const { return elapse_us(start_, SteadyClock::now()); }
  void reset() { start_ = SteadyClock::now(); }

 private:
  Timepoint start_;
};

// Monotone counter: wait(c) blocks until the counter exceeds c (role of SyncSemaphore,
// kvtransfer/src/semaphore.cpp:5-25).  wait_for adds a deadline so no thread waits forever
// on a peer that went away.
class SyncSemaphore {
 public:
  void wait(uint32_t cond);
  bool wait_for(uint32_t cond, std::chrono::milliseconds timeout);
  void release();                    // counter += 1
  uint32_t release(uint32_t cond);   // counter = max(counter, cond); returns the new value
  uint32_t value();

 private:
  alignas(64) std::mutex mu_;
  std::condition_variable cv_;
  uint32_t ready_{0};
  std::atomic<uint32_t> fast_{0};   // mirror of ready_ for the short spin before blocking
};

// FIFO pool.  spawn(fn) runs on any worker; spawn(fn, hint) pins all tasks with the same hint
// to one worker so they execute in submission order (one destination's batches stay ordered,
// as the reference gets from its thread_hint, kvtransfer/src/client.cpp:94-104).
class ThreadPool {
 public:
  explicit ThreadPool(size_t n, std::string name = "kvx");
  ~ThreadPool();
  ThreadPool(const ThreadPool&) = delete;
  void spawn(std::function<void()> fn);
  void spawn(std::function<void()> fn, int hint);
  size_t size() const { return workers_.size(); }
  void drain();  // block until every queued task has finished

 private:
  struct Worker {
    std::mutex mu;
    std::condition_variable cv;
    std::deque<std::function<void()>> q;
    std::thread thd;
    bool busy{false};
    std::atomic<uint32_t> pending{0};   // queued + running tasks; drain() polls it before it blocks
  };
  void run(Worker* w, size_t idx);
  std::vector<std::unique_ptr<Worker>> workers_;
  std::atomic<size_t> rr_{0};
  std::atomic<bool> stop_{false};
  std::string name_;
};

template <typename T>
class BlockingQueue {
 public:
  void push(T v) {
    {
      std::lock_guard<std::mutex> g(mu_);
      q_.emplace_back(std::move(v));
    }
    cv_.notify_one();
  }
  T pop() {
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [this] { return !q_.empty(); });
    T v = std::move(q_.front());
    q_.pop_front();
    return v;
  }
  std::optional<T> pop_for(std::chrono::milliseconds d) {
    std::unique_lock<std::mutex> lk(mu_);
    if (!cv_.wait_for(lk, d, [this] { return !q_.empty(); })) return std::nullopt;
    T v = std::move(q_.front());
    q_.pop_front();
    return v;
  }
  size_t size() {
    std::lock_guard<std::mutex> g(mu_);
    return q_.size();
  }

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<T> q_;
};

// ---- sockets ------------------------------------------------------------------------------
class FdGuard {
 public:
  FdGuard() = default;
  explicit FdGuard(int fd) : fd_(fd) {}
  FdGuard(FdGuard&& o) noexcept : fd_(o.fd_) { o.fd_ = -1; }
  FdGuard& operator=(FdGuard&& o) noexcept;
  FdGuard(const FdGuard&) = delete;
  ~FdGuard();
  int fd() const { return fd_; }
  bool valid() const { return fd_ >= 0; }
  int release() {
    int f = fd_;
    fd_ = -1;
    return f;
  }
  void reset();

 private:
  int fd_{-1};
};

// All helpers return -1 on error (errno set) and never block past timeout_ms (<=0: no limit).
int tcp_connect(const std::string& ip, int port, int timeout_ms);
int tcp_listen(const std::string& ip, int port, int backlog, int* bound_port);
ssize_t write_full(int fd, const void* buf, size_t len, int timeout_ms);
ssize_t read_full(int fd, void* buf, size_t len, int timeout_ms);
std::string local_ip();  // VLLM_HOST_IP, else the address a UDP "connect" would use

}  // namespace kvx
