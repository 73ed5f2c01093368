// gdrcopy shim: maps GPU memory into the CPU's address space through libgdrapi when that
// library and its kernel module are present.  The reference uses it to CRC-check what an RDMA
// write delivered (kvtransfer/src/gdr.cpp:46-286, rdma_channel.cpp:143-296).  libgdrapi is
// resolved with dlopen at first use; without it every call reports "unavailable" and callers
// fall back to a device-to-host copy.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <string>

namespace kvx {

class GdrMapping {
 public:
  GdrMapping() = default;
  ~GdrMapping();
  GdrMapping(const GdrMapping&) = delete;
  GdrMapping& operator=(const GdrMapping&) = delete;
  // Pins and maps [dev_ptr, dev_ptr + bytes); false (with why()) when gdrcopy is unavailable.
  bool map(uint64_t dev_ptr, size_t bytes);
  void unmap();
  const void* cpu_ptr() const { return cpu_; }
  const std::string& why() const { return why_; }

 private:
  void* handle_ = nullptr;   // gdr_t
  uint64_t mh_[4] = {0, 0, 0, 0};   // gdr_mh_t is a small opaque struct
  void* map_base_ = nullptr;
  void* cpu_ = nullptr;
  size_t map_bytes_ = 0;
  std::string why_;
};

bool gdr_available(std::string* why);
// CRC-32 (zlib polynomial) of a host buffer; used for end-to-end transfer checks.
uint32_t crc32_bytes(const void* data, size_t n, uint32_t seed = 0);

}  // namespace kvx
