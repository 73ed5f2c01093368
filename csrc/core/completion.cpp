#include "core/completion.h"

#include <pthread.h>

#include <vector>

#include "core/log.h"

namespace kvx {

CompletionPoller& CompletionPoller::instance() {
  static CompletionPoller* p = new CompletionPoller();   // lives for the process: batches may finish during exit
  return *p;
}

CompletionPoller::CompletionPoller() : thd_([this] { run(); }) {}

CompletionPoller::~CompletionPoller() {
  {
    std::lock_guard<std::mutex> g(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  if (thd_.joinable()) thd_.join();
}

void CompletionPoller::add(Entry e) {
  {
    std::lock_guard<std::mutex> g(mu_);
    entries_.emplace_back(std::move(e));
  }
  cv_.notify_one();
}

size_t CompletionPoller::pending() {
  std::lock_guard<std::mutex> g(mu_);
  return entries_.size() + in_finish_;
}

bool CompletionPoller::drain(std::chrono::milliseconds timeout) {
  std::unique_lock<std::mutex> lk(mu_);
  return idle_cv_.wait_for(lk, timeout, [this] { return entries_.empty() && in_finish_ == 0; });
}

void CompletionPoller::run() {
  pthread_setname_np(pthread_self(), "kvtcomplete");
  std::vector<Entry> ready;
  std::vector<PollResult> results;
  std::vector<const void*> blocked;
  int idle_rounds = 0;
  for (;;) {
    {
      std::unique_lock<std::mutex> lk(mu_);
      if (entries_.empty() && in_finish_ == 0) idle_cv_.notify_all();
      cv_.wait(lk, [this] { return stop_ || !entries_.empty(); });
      if (stop_ && entries_.empty()) return;
      // poll the first entry of every owner; later entries of an owner wait their turn
      blocked.clear();
      const Timepoint now = SteadyClock::now();
      for (auto it = entries_.begin(); it != entries_.end();) {
        bool owner_blocked = false;
        for (const void* o : blocked) owner_blocked = owner_blocked || o == it->owner;
        if (owner_blocked) {
          ++it;
          continue;
        }
        PollResult r = PollResult::FAILED;
        try {
          r = it->poll();
        } catch (const std::exception& ex) {
          LOG(ERROR) << "completion poll failed: " << ex.what();
        }
        if (r == PollResult::PENDING && now > it->deadline) {
          LOG(ERROR) << "completion record did not arrive before its deadline";
          r = PollResult::FAILED;
        }
        if (r == PollResult::PENDING) {
          blocked.push_back(it->owner);
          ++it;
        } else {
          ready.emplace_back(std::move(*it));
          results.push_back(r);
          it = entries_.erase(it);
        }
      }
      in_finish_ += ready.size();
    }
    if (!ready.empty()) {
      for (size_t i = 0; i < ready.size(); ++i) {
        try {
          ready[i].finish(results[i]);
        } catch (const std::exception& ex) {
          LOG(ERROR) << "completion handler failed: " << ex.what();
        }
      }
      {
        std::lock_guard<std::mutex> g(mu_);
        in_finish_ -= ready.size();
        if (entries_.empty() && in_finish_ == 0) idle_cv_.notify_all();
      }
      ready.clear();
      results.clear();
      idle_rounds = 0;
      continue;
    }
    // nothing arrived: a short spin keeps the latency of a record that is about to land in the microseconds,
    // then back off so that a long transfer does not cost a core
    if (++idle_rounds < 200) {
      std::this_thread::yield();
    } else {
      std::this_thread::sleep_for(std::chrono::microseconds(idle_rounds < 2000 ? 5 : 50));
    }
  }
}

void InflightCounter::done(bool ok) {
  if (!ok) failed_.fetch_add(1, std::memory_order_release);
  done_.fetch_add(1, std::memory_order_release);
  std::lock_guard<std::mutex> g(mu_);
  cv_.notify_all();
}

uint64_t InflightCounter::inflight() const {
  const uint64_t d = done_.load(std::memory_order_acquire);
  const uint64_t s = submitted_.load(std::memory_order_relaxed);
  return s > d ? s - d : 0;
}

bool InflightCounter::wait_at_most(uint64_t max_inflight, std::chrono::milliseconds timeout) {
  // the common case resolves within a transfer's duration: spin briefly before sleeping on the condition
  for (int i = 0; i < 2000; ++i) {
    if (inflight() <= max_inflight) return true;
    std::this_thread::yield();
  }
  std::unique_lock<std::mutex> lk(mu_);
  return cv_.wait_for(lk, timeout, [&] { return inflight() <= max_inflight; });
}

}  // namespace kvx
