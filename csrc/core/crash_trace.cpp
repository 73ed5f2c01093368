#include "core/crash_trace.h"

#include <execinfo.h>
#include <signal.h>
#include <stdlib.h>
#include <string.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>

namespace kvx {

namespace {

constexpr int kSignals[] = {SIGSEGV, SIGBUS, SIGFPE, SIGILL, SIGABRT};
struct sigaction g_prev[sizeof(kSignals) / sizeof(kSignals[0])];
std::atomic<bool> g_installed{false};

void put_str(const char* s) {
  const ssize_t r = write(2, s, strlen(s));
  (void)r;
}

void put_num(long v) {
  char buf[24];
  int i = 23;
  buf[i] = '\0';
  const bool neg = v < 0;
  unsigned long u = neg ? 0ul - static_cast<unsigned long>(v) : static_cast<unsigned long>(v);
  do {
    buf[--i] = static_cast<char>('0' + u % 10);
    u /= 10;
  } while (u != 0 && i > 1);
  if (neg) buf[--i] = '-';
  put_str(buf + i);
}

void on_fatal(int sig, siginfo_t* info, void* uctx) {
  put_str("\n==== kvtransfer crash trace: signal ");
  put_num(sig);
  put_str(" in thread ");
  put_num(static_cast<long>(syscall(SYS_gettid)));
  put_str(" ====\n");
  void* frames[64];
  const int n = backtrace(frames, 64);
  backtrace_symbols_fd(frames, n, 2);
  put_str("==== end of trace ====\n");
  // hand over to the handler that was there before (the interpreter's fault handler, or the default action)
  for (size_t i = 0; i < sizeof(kSignals) / sizeof(kSignals[0]); ++i) {
    if (kSignals[i] != sig) continue;
    const struct sigaction& prev = g_prev[i];
    if ((prev.sa_flags & SA_SIGINFO) != 0 && prev.sa_sigaction != nullptr) {
      prev.sa_sigaction(sig, info, uctx);
      return;
    }
    if (prev.sa_handler != SIG_DFL && prev.sa_handler != SIG_IGN && prev.sa_handler != nullptr) {
      prev.sa_handler(sig);
      return;
    }
  }
  signal(sig, SIG_DFL);
  raise(sig);
}

}  // namespace

bool install_crash_trace(bool force) {
  if (!force) {
    const char* v = getenv("BLLM_KVTRANS_CRASH_TRACE");
    if (v == nullptr || v[0] == '\0' || v[0] == '0') return false;
  }
  if (g_installed.exchange(true)) return true;
  void* warm[2];
  backtrace(warm, 2);      // the first call loads the unwinder: not something to do inside a signal handler
  for (size_t i = 0; i < sizeof(kSignals) / sizeof(kSignals[0]); ++i) {
    struct sigaction sa;
    memset(&sa, 0, sizeof(sa));
    sa.sa_sigaction = on_fatal;
    sa.sa_flags = SA_SIGINFO | SA_NODEFER;
    sigemptyset(&sa.sa_mask);
    sigaction(kSignals[i], &sa, &g_prev[i]);
  }
  return true;
}

}  // namespace kvx
