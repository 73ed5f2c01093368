#include "core/gdr.h"

#include <dlfcn.h>

#include <mutex>

namespace kvx {

namespace {
struct GdrMh {
  unsigned long h;
};
struct Api {
  void* lib = nullptr;
  void* (*open)() = nullptr;
  int (*close)(void*) = nullptr;
  int (*pin_buffer)(void*, unsigned long, size_t, uint64_t, uint32_t, GdrMh*) = nullptr;
  int (*unpin_buffer)(void*, GdrMh) = nullptr;
  int (*map)(void*, GdrMh, void**, size_t) = nullptr;
  int (*unmap)(void*, GdrMh, void*, size_t) = nullptr;
  std::string why;
};

Api& api() {
  static Api a;
  static std::once_flag once;
  std::call_once(once, [] {
    a.lib = dlopen("libgdrapi.so.2", RTLD_NOW | RTLD_LOCAL);
    if (a.lib == nullptr) a.lib = dlopen("libgdrapi.so", RTLD_NOW | RTLD_LOCAL);
    if (a.lib == nullptr) {
      a.why = "libgdrapi not found";
      return;
    }
    a.open = reinterpret_cast<decltype(a.open)>(dlsym(a.lib, "gdr_open"));
    a.close = reinterpret_cast<decltype(a.close)>(dlsym(a.lib, "gdr_close"));
    a.pin_buffer = reinterpret_cast<decltype(a.pin_buffer)>(dlsym(a.lib, "gdr_pin_buffer"));
    a.unpin_buffer = reinterpret_cast<decltype(a.unpin_buffer)>(dlsym(a.lib, "gdr_unpin_buffer"));
    a.map = reinterpret_cast<decltype(a.map)>(dlsym(a.lib, "gdr_map"));
    a.unmap = reinterpret_cast<decltype(a.unmap)>(dlsym(a.lib, "gdr_unmap"));
    if (!a.open || !a.close || !a.pin_buffer || !a.unpin_buffer || !a.map || !a.unmap) {
      a.why = "libgdrapi lacks an expected symbol";
      a.open = nullptr;
    }
  });
  return a;
}

constexpr uint64_t kGpuPage = 64 * 1024;
}  // namespace

bool gdr_available(std::string* why) {
  Api& a = api();
  if (a.open == nullptr) {
    if (why != nullptr) *why = a.why;
    return false;
  }
  return true;
}

bool GdrMapping::map(uint64_t dev_ptr, size_t bytes) {
  unmap();
  Api& a = api();
  if (a.open == nullptr) {
    why_ = a.why;
    return false;
  }
  handle_ = a.open();
  if (handle_ == nullptr) {
    why_ = "gdr_open failed (gdrdrv kernel module not loaded?)";
    return false;
  }
  const uint64_t base = dev_ptr & ~(kGpuPage - 1);
  map_bytes_ = static_cast<size_t>(((dev_ptr + bytes + kGpuPage - 1) & ~(kGpuPage - 1)) - base);
  GdrMh mh{};
  if (a.pin_buffer(handle_, base, map_bytes_, 0, 0, &mh) != 0) {
    why_ = "gdr_pin_buffer failed";
    a.close(handle_);
    handle_ = nullptr;
    return false;
  }
  mh_[0] = mh.h;
  if (a.map(handle_, mh, &map_base_, map_bytes_) != 0) {
    why_ = "gdr_map failed";
    a.unpin_buffer(handle_, mh);
    a.close(handle_);
    handle_ = nullptr;
    return false;
  }
  cpu_ = static_cast<char*>(map_base_) + (dev_ptr - base);
  return true;
}

void GdrMapping::unmap() {
  if (handle_ == nullptr) return;
  Api& a = api();
  GdrMh mh{static_cast<unsigned long>(mh_[0])};
  if (map_base_ != nullptr) a.unmap(handle_, mh, map_base_, map_bytes_);
  a.unpin_buffer(handle_, mh);
  a.close(handle_);
  handle_ = map_base_ = cpu_ = nullptr;
}

GdrMapping::~GdrMapping() { unmap(); }

uint32_t crc32_bytes(const void* data, size_t n, uint32_t seed) {
  static uint32_t table[256];
  static std::once_flag once;
  std::call_once(once, [] {
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
      table[i] = c;
    }
  });
  uint32_t c = ~seed;
  const unsigned char* p = static_cast<const unsigned char*>(data);
  for (size_t i = 0; i < n; ++i) c = table[(c ^ p[i]) & 0xFF] ^ (c >> 8);
  return ~c;
}

}  // namespace kvx
