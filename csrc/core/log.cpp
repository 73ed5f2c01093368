#include "core/log.h"

#include <sys/syscall.h>
#include <sys/time.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace kvx {

static int env_int(const char* name, int def) {
  const char* v = getenv(name);
  if (v == nullptr || *v == '\0') return def;
  return atoi(v);
}

int min_log_level() {
  static int lvl = env_int("LLMOPS_CPP_MIN_LOG_LEVEL", 1);
  return lvl;
}

int max_vlog_level() {
  static int lvl = env_int("LLMOPS_CPP_MAX_VLOG_LEVEL", 0);
  return lvl;
}

static std::atomic<void (*)(int, const std::string&)> g_sink{nullptr};

void set_log_sink(void (*sink)(int, const std::string&)) { g_sink.store(sink); }

LogMessage::LogMessage(const char* file, int line, int level) : file_(file), line_(line), level_(level) {}

LogMessage::~LogMessage() {
  static const char kLevel[] = {'I', 'W', 'E', 'F'};
  const char* base = strrchr(file_, '/');
  base = base ? base + 1 : file_;
  struct timeval tv;
  gettimeofday(&tv, nullptr);
  struct tm tmv;
  time_t sec = tv.tv_sec;
  localtime_r(&sec, &tmv);
  char head[128];
  snprintf(head, sizeof(head), "%04d-%02d-%02d %02d:%02d:%02d.%06ld:%d:%ld %c %s:%d] ", tmv.tm_year + 1900,
           tmv.tm_mon + 1, tmv.tm_mday, tmv.tm_hour, tmv.tm_min, tmv.tm_sec, (long)tv.tv_usec, (int)getpid(),
           (long)syscall(SYS_gettid), kLevel[level_ & 3], base, line_);
  std::string line = std::string(head) + ss_.str();
  auto sink = g_sink.load();
  if (sink != nullptr) {
    sink(level_, line);
  } else {
    line.push_back('\n');
    fwrite(line.data(), 1, line.size(), stderr);
  }
  if (level_ == LOG_FATAL) abort();
}

}  // namespace kvx
