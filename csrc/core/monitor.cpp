#include "core/monitor.h"

#include <dlfcn.h>
#include <malloc.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <mutex>
#include <sstream>
#include <thread>

#include "core/envcfg.h"
#include "core/log.h"
#include "core/util.h"

namespace kvx {

namespace {
using mallctl_t = int(const char*, void*, size_t*, void*, size_t);
mallctl_t* g_mallctl = nullptr;
std::once_flag g_once;
std::atomic<int> g_port{0};
std::atomic<bool> g_stop{false};
std::thread g_thread;
std::mutex g_mu;

void resolve_mallctl() {
  std::call_once(g_once, [] { g_mallctl = reinterpret_cast<mallctl_t*>(dlsym(RTLD_DEFAULT, "mallctl")); });
}

int set_prof_active(bool on) {
  resolve_mallctl();
  if (g_mallctl == nullptr) return -33;
  bool old = false;
  size_t len = sizeof(old);
  if (g_mallctl("prof.active", &old, &len, &on, sizeof(on)) != 0) return -34;
  return old ? 1 : 0;
}

std::string first_word(const std::string& s) {
  size_t a = s.find_first_not_of(" \t\r\n");
  if (a == std::string::npos) return "";
  size_t b = s.find_first_of(" \t\r\n", a);
  return s.substr(a, b == std::string::npos ? std::string::npos : b - a);
}

std::string dump_heap(const std::string& path) {
  if (path.empty()) return "empty filepath\n";
  resolve_mallctl();
  if (g_mallctl != nullptr) {
    const char* p = path.c_str();
    return g_mallctl("prof.dump", nullptr, nullptr, &p, sizeof(p)) == 0 ? "ok\n" : "error\n";
  }
  FILE* f = fopen(path.c_str(), "w");
  if (f == nullptr) return "error\n";
  const int rc = malloc_info(0, f);   // glibc: per-arena XML
  fclose(f);
  return rc == 0 ? "ok\n" : "error\n";
}

std::string process_stats() {
  std::ostringstream ss;
  long rss_pages = 0, vm_pages = 0;
  if (FILE* f = fopen("/proc/self/statm", "r")) {
    if (fscanf(f, "%ld %ld", &vm_pages, &rss_pages) != 2) rss_pages = vm_pages = 0;
    fclose(f);
  }
  const long page = sysconf(_SC_PAGESIZE);
  struct mallinfo2 mi = mallinfo2();
  ss << "pid=" << getpid() << " rss_bytes=" << rss_pages * page << " vm_bytes=" << vm_pages * page
     << " malloc_in_use=" << mi.uordblks << " malloc_free=" << mi.fordblks << " malloc_mmap=" << mi.hblkhd
     << " jemalloc=" << (g_mallctl != nullptr ? 1 : 0) << "\n";
  return ss.str();
}

void serve(int listen_fd) {
  FdGuard guard(listen_fd);
  while (!g_stop.load()) {
    pollfd pfd{listen_fd, POLLIN, 0};
    if (poll(&pfd, 1, 200) <= 0) continue;
    int conn = accept(listen_fd, nullptr, nullptr);
    if (conn < 0) continue;
    FdGuard cg(conn);
    char buf[1024];
    std::string pending;
    while (!g_stop.load()) {
      pollfd cp{conn, POLLIN, 0};
      if (poll(&cp, 1, 200) <= 0) continue;
      const ssize_t n = read(conn, buf, sizeof(buf));
      if (n <= 0) break;
      pending.append(buf, static_cast<size_t>(n));
      size_t nl;
      bool quit = false;
      while ((nl = pending.find('\n')) != std::string::npos) {
        const std::string line = pending.substr(0, nl);
        pending.erase(0, nl + 1);
        if (first_word(line) == "quit") {
          quit = true;
          break;
        }
        const std::string out = monitor_handle_line(line);
        if (!out.empty() && write(conn, out.data(), out.size()) < 0) quit = true;
      }
      if (quit) break;
    }
  }
}
}  // namespace

std::string monitor_handle_line(const std::string& line) {
  static const char kActive[] = "prof active", kDeactive[] = "prof deactive", kDump[] = "prof dump ";
  if (line.compare(0, sizeof(kDeactive) - 1, kDeactive) == 0) return "prev=" + std::to_string(set_prof_active(false)) + "\n";
  if (line.compare(0, sizeof(kActive) - 1, kActive) == 0) return "prev=" + std::to_string(set_prof_active(true)) + "\n";
  if (line.compare(0, sizeof(kDump) - 1, kDump) == 0) return dump_heap(first_word(line.substr(sizeof(kDump) - 1)));
  const std::string w = first_word(line);
  if (w == "stats") {
    resolve_mallctl();
    return process_stats();
  }
  if (w == "env") return envcfg_dump();
  return w.empty() ? "" : "unknown command\n";
}

int monitor_start() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_port.load() != 0) return g_port.load();
  int port = 0;
  const int fd = tcp_listen("0.0.0.0", 0, 7, &port);
  if (fd < 0) {
    LOG(ERROR) << "monitor: cannot listen, errno=" << errno;
    return 0;
  }
  resolve_mallctl();
  if (env_heap_prof() && g_mallctl != nullptr) LOG(INFO) << "monitor: prof active. prev=" << set_prof_active(true);
  g_stop.store(false);
  g_thread = std::thread(serve, fd);
  g_port.store(port);
  LOG(INFO) << "monitor listen=0.0.0.0:" << port;
  return port;
}

void monitor_stop() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_port.load() == 0) return;
  g_stop.store(true);
  if (g_thread.joinable()) g_thread.join();
  g_port.store(0);
}

int monitor_port() { return g_port.load(); }

}  // namespace kvx
