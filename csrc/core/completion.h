// Asynchronous completion of batches on device transports.
//
// A device transport does not make a host thread wait for the GPU: its flush enqueues a completion
// record behind the batch (a kernel that writes sequence number, status words and timer stamps into
// mapped host memory) and returns a ticket.  CompletionPoller is the one thread per process that
// turns arrived records into the engine's "batch finished" work: request states, the send-done RPC
// to the scheduler (same wire format as the synchronous path, kvtransfer/src/tx_stub.cpp:324-386),
// step metrics.  Entries of one owner (a send stub) complete in the order they were added; an entry
// that does not complete before its deadline is finished as failed, never waited for without limit.
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>
#include <thread>

#include "core/util.h"

namespace kvx {

enum class PollResult { PENDING, DONE, FAILED };

class CompletionPoller {
 public:
  struct Entry {
    const void* owner = nullptr;                 // entries of one owner finish in order
    std::function<PollResult()> poll;            // non-blocking
    std::function<void(PollResult)> finish;      // DONE or FAILED (also FAILED when the deadline passed)
    Timepoint deadline;
  };
  static CompletionPoller& instance();
  void add(Entry e);
  size_t pending();
  // Blocks until nothing is pending or the timeout ran out; returns true when idle.
  bool drain(std::chrono::milliseconds timeout);
  ~CompletionPoller();

 private:
  CompletionPoller();
  void run();
  std::mutex mu_;
  std::condition_variable cv_, idle_cv_;
  std::deque<Entry> entries_;
  size_t in_finish_{0};
  bool stop_{false};
  std::thread thd_;
};

// Batches in flight of one client: counted when a step hands them to the sender threads, released
// when their completion has been processed.  Lets the engine thread bound how far it runs ahead of
// the transfers without synchronising a stream.
class InflightCounter {
 public:
  void add(uint64_t n) { submitted_.fetch_add(n, std::memory_order_relaxed); }
  void done(bool ok = true);
  uint64_t inflight() const;
  uint64_t finished() const { return done_.load(std::memory_order_acquire); }
  uint64_t failed() const { return failed_.load(std::memory_order_acquire); }   // finished batches that did not arrive
  // Waits until at most `max_inflight` batches are outstanding; false when the timeout ran out.
  bool wait_at_most(uint64_t max_inflight, std::chrono::milliseconds timeout);

 private:
  std::atomic<uint64_t> submitted_{0}, done_{0}, failed_{0};
  std::mutex mu_;
  std::condition_variable cv_;
};

}  // namespace kvx
