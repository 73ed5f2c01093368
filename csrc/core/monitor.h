// Process monitor: a line protocol on an ephemeral TCP port for looking inside a running engine.
//
// Commands (one per line), same shape as the reference's monitor
// (kvtransfer/src/monitor.cpp:23-165: "prof active", "prof deactive", "prof dump <file>" drive
// jemalloc's heap profiler through mallctl when jemalloc is the process allocator):
//   prof active | prof deactive     -> "prev=<0|1>", or "prev=-33" when no jemalloc is loaded
//   prof dump <file>                -> jemalloc heap profile, or glibc malloc_info XML when there
//                                      is no jemalloc; "ok" / "error"
//   stats                           -> one line of key=value process figures (rss, arena bytes)
//   env                             -> the engine's resolved environment settings
//   quit                            -> closes the connection
// Nothing is started unless monitor_start() is called (the Python package does so when
// BLLM_KVTRANS_MONITOR=1).
#pragma once
#include <string>

namespace kvx {

// Starts the monitor thread once per process and returns the port it listens on (0 on failure).
int monitor_start();
void monitor_stop();
int monitor_port();
// The command interpreter, exposed for tests: returns what would be written back.
std::string monitor_handle_line(const std::string& line);

}  // namespace kvx
