// Minimal glog-style logging for the native engine.
// Same knobs and line format as the reference logger (kvtransfer/src/third_party/logging.cpp:
// 106-147): LLMOPS_CPP_MIN_LOG_LEVEL (0=INFO,1=WARNING,2=ERROR,3=FATAL), LLMOPS_CPP_VMODULE-less
// VLOG via LLMOPS_CPP_MAX_VLOG_LEVEL, stderr line `time.us:pid:tid L file:line] msg`.
#pragma once
#include <sstream>
#include <string>

namespace kvx {

enum LogLevel { LOG_INFO = 0, LOG_WARNING = 1, LOG_ERROR = 2, LOG_FATAL = 3 };

int min_log_level();
int max_vlog_level();
// Test hook: capture log lines instead of writing stderr (nullptr restores stderr).
void set_log_sink(void (*sink)(int level, const std::string& line));

class LogMessage {
 public:
  LogMessage(const char* file, int line, int level);
  ~LogMessage();
  std::ostream& stream() { return ss_; }

 private:
  std::ostringstream ss_;
  const char* file_;
  int line_;
  int level_;
};

struct LogVoidify {
  void operator&(std::ostream&) {}
};

}  // namespace kvx

#define KVX_LOG_IS_ON(lvl) ((lvl) >= ::kvx::min_log_level())
#define LOG(severity)                                   \
  !KVX_LOG_IS_ON(::kvx::LOG_##severity) ? (void)0       \
      : ::kvx::LogVoidify() & ::kvx::LogMessage(__FILE__, __LINE__, ::kvx::LOG_##severity).stream()
#define VLOG(n)                                 \
  ((n) > ::kvx::max_vlog_level()) ? (void)0     \
      : ::kvx::LogVoidify() & ::kvx::LogMessage(__FILE__, __LINE__, ::kvx::LOG_INFO).stream()
