#include "core/fault_inject.h"

#include <atomic>
#include <chrono>
#include <random>
#include <stdexcept>
#include <thread>

#include "core/envcfg.h"

namespace kvx {

static std::atomic<int> g_countdown{0};

static bool roll() {
  const int rate = env_debug_tx_failrate() - 1;
  if (rate <= 0) return false;
  thread_local std::mt19937 rng{std::random_device{}()};
  return static_cast<int>(rng() % 100) < rate;
}

void fault_inject_arm(int throw_after_n) { g_countdown.store(throw_after_n > 0 ? throw_after_n : 0); }

void fault_inject_throw() {
  int c = g_countdown.load();
  while (c > 0) {
    if (g_countdown.compare_exchange_weak(c, c - 1)) {
      if (c == 1) throw std::runtime_error("fault_inject: armed failure");
      break;
    }
  }
  if (roll()) throw std::runtime_error("fault_inject: random failure");
}

static std::atomic<int> g_drop_completions{0};

void fault_inject_arm_drop_completion(int n) { g_drop_completions.store(n > 0 ? n : 0); }

bool fault_inject_drop_completion() {
  int c = g_drop_completions.load();
  while (c > 0) {
    if (g_drop_completions.compare_exchange_weak(c, c - 1)) return true;
  }
  return false;
}

static std::atomic<int> g_corrupt_checks{0};

void fault_inject_arm_corrupt_check(int n) { g_corrupt_checks.store(n > 0 ? n : 0); }

bool fault_inject_corrupt_check() {
  int c = g_corrupt_checks.load();
  while (c > 0) {
    if (g_corrupt_checks.compare_exchange_weak(c, c - 1)) return true;
  }
  return false;
}

void fault_inject_sleep(int max_us) {
  if (max_us <= 0 || !roll()) return;
  const int delay_ms = env_debug_tx_delay_ms();
  int us = delay_ms > 1 ? delay_ms * 1000 : max_us;
  std::this_thread::sleep_for(std::chrono::microseconds(us));
}

}  // namespace kvx
