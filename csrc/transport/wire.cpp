#include "transport/wire.h"

#include <unistd.h>

#include <fstream>
#include <functional>

#include "core/util.h"

namespace kvx {

bool send_frame(int fd, const void* payload, size_t len, int timeout_ms) {
  return send_frame2(fd, payload, len, nullptr, 0, timeout_ms);
}

bool send_frame2(int fd, const void* head, size_t head_len, const void* body, size_t body_len, int timeout_ms) {
  const uint64_t total = head_len + body_len;
  if (total > 0xffffffffull) return false;
  const uint32_t n = static_cast<uint32_t>(total);
  if (write_full(fd, &n, 4, timeout_ms) != 4) return false;
  if (head_len && write_full(fd, head, head_len, timeout_ms) != static_cast<ssize_t>(head_len)) return false;
  if (body_len && write_full(fd, body, body_len, timeout_ms) != static_cast<ssize_t>(body_len)) return false;
  return true;
}

bool recv_frame(int fd, std::string& buf, int timeout_ms) {
  uint32_t n = 0;
  if (read_full(fd, &n, 4, timeout_ms) != 4) return false;
  buf.resize(n);
  if (n == 0) return true;
  return read_full(fd, buf.data(), n, timeout_ms) == static_cast<ssize_t>(n);
}

std::string PeerMemInfo::serialize() const {
  std::string s;
  put(s, pid);
  put(s, device);
  put(s, host_id);
  put(s, num_layers);
  put(s, num_tensors);
  for (const auto& t : tensors) {
    put(s, t.ptr);
    put(s, t.alloc_base);
    s.append(t.ipc_handle, 64);
    put(s, t.has_handle);
  }
  return s;
}

bool PeerMemInfo::parse(const char* p, size_t len, PeerMemInfo* out) {
  const char* end = p + len;
  if (!take(p, end, &out->pid) || !take(p, end, &out->device) || !take(p, end, &out->host_id) ||
      !take(p, end, &out->num_layers) || !take(p, end, &out->num_tensors))
    return false;
  const size_t n = static_cast<size_t>(out->num_layers) * out->num_tensors;
  if (n > (1u << 20)) return false;
  out->tensors.resize(n);
  for (auto& t : out->tensors) {
    if (!take(p, end, &t.ptr) || !take(p, end, &t.alloc_base)) return false;
    if (static_cast<size_t>(end - p) < 65) return false;
    memcpy(t.ipc_handle, p, 64);
    p += 64;
    t.has_handle = static_cast<uint8_t>(*p++);
  }
  return true;
}

uint64_t this_host_id() {
  static uint64_t id = [] {
    std::ifstream f("/proc/sys/kernel/random/boot_id");
    std::string s;
    if (f) std::getline(f, s);
    char host[256] = {0};
    gethostname(host, sizeof(host) - 1);
    s += host;
    return static_cast<uint64_t>(std::hash<std::string>{}(s)) | 1ull;
  }();
  return id;
}

}  // namespace kvx
